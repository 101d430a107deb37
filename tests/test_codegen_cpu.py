"""CPU tests of the template instantiator's host logic: graphs are compiled through the
backend registered for the *cpu* device in dry-run mode, so the generated CUDA source is
produced and cross-compiled with nvcc for sm_100a but never launched.  What is checked is
classification (which template, how many kernels), the index analysis and the launch
chooser - not numerics, which need a GPU (tests/test_compile_gpu.py)."""
import os
import re
import shutil

import pytest
import sympy
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.skipif(shutil.which("nvcc") is None, reason="nvcc not available")


def launch_shape(code):
    """(team, teams, vpt) a generated row module names as its default launch shape."""
    return tuple(int(re.search(rf"#define IXB_ROW_{m} (\d+)", code).group(1)) for m in ("TEAM", "TEAMS", "VPT"))


def generated(fn, *args):
    from torch._inductor.utils import run_and_get_code

    torch._dynamo.reset()
    _, code = run_and_get_code(torch.compile(fn), *args)
    return "\n".join(code)


def test_c1_graph_is_one_row_kernel(dry_backend):
    code = generated(lambda x, w, b: F.gelu(x * w + b).sum(-1), torch.randn(64, 1024), torch.randn(1024),
                     torch.randn(1024))
    assert code.count("ixb_load_kernel('''") == 1
    assert launch_shape(code) == (128, 1, 2)              # 1024 fp32 = 256 vectors
    # w and b are the same for every row: loaded once per thread; x is fetched a row ahead
    assert code.count("kinit<0, IXB_ROW_KREGS>(c, k.k0,") == 1 and code.count("kinit<1, IXB_ROW_KREGS>(c, k.k1,") == 1
    assert "#define IXB_ROW_KREGS 2" in code             # both stay in registers at 8 elements per thread
    assert "c.fetch_row(" in code and "c.template operand<STAGED, float>(raw.s0" in code
    # x * w + b is one fused multiply-add, the decomposed exact GELU one call
    assert "ixb::gen::op::fma(" in code and "ixb::gen::op::gelu_erf(" in code
    assert "reduce<ixb::SumOp>" in code
    assert "triton_" not in code


def test_c2_chain_is_one_row_kernel_with_four_reductions(dry_backend):
    fn = lambda x, g, ga, be: F.layer_norm(torch.softmax(x, -1) * g + x, (4096,), ga, be, 1e-5)
    code = generated(fn, torch.randn(32, 4096).bfloat16(), *(torch.randn(4096).bfloat16() for _ in range(3)))
    assert code.count("ixb_load_kernel('''") == 1
    assert launch_shape(code) == (256, 1, 2)              # 4096 bf16 = 512 vectors
    # two exchanges per row: the online softmax, which also carries sum(e * g) and sum(x) for
    # the LayerNorm mean, and the centred second moment
    assert ("c.template online_softmax<1, 1>(tmp1, ixb::gen::refs<kN>(ixb::gen::kget<0, IXB_ROW_KREGS>(c, k.k0)), "
            "ixb::gen::refs<kN>(tmp0))") in code
    # g is used twice (rider and product), so it is operand 0: the last to leave the registers
    assert code.count("kget<0, IXB_ROW_KREGS>") == 2 and "#define IXB_ROW_KREGS 3" in code
    assert ".scaled[0]" in code and ".plain[0]" in code
    assert len(re.findall(r"c\.template reduce<", code)) == 0 and code.count("c.reduce_dot(") == 1
    # exp(x - max) / sum comes from the exponentials the exchange kept
    assert re.search(r"op::mul\(tmp\d+\.e, ixb::gen::op::truediv\(tmp\d+\.r, tmp\d+\)\)", code)
    assert "c.prefetch_row(" in code
    assert "c.template put_row<STAGED>(" in code
    assert "tune=dict(" in code and "idempotent=True" in code


def test_c2_chain_with_two_pass_softmax(dry_backend):
    """The same chain with the merged exchange switched off: four plain reductions."""
    from inductor_x_b200 import config

    fn = lambda x, g, ga, be: F.layer_norm(torch.softmax(x, -1) * g + x, (4096,), ga, be, 1e-5)
    config.merged_online_softmax = False
    try:
        code = generated(fn, torch.randn(32, 4096).bfloat16(), *(torch.randn(4096).bfloat16() for _ in range(3)))
    finally:
        config.merged_online_softmax = True
    assert len(re.findall(r"c\.template reduce<", code)) + code.count("c.reduce_dot(") == 4
    assert "exp_sub(" in code          # exp(x - rowmax) as one packed fma and the exponential


def test_integer_reductions_are_exact_by_construction(dry_backend):
    code = generated(lambda t: (t.sum(-1), t.amax(-1)), torch.randint(0, 1 << 40, (16, 1000)))
    assert "reduce_int<typename Ctx::ISum>" in code and "reduce_int<typename Ctx::IMax>" in code
    assert "to_int(c.template reduce<" not in code
    code = generated(lambda t: t.sum(0), torch.randint(0, 1 << 40, (256, 1024)))
    assert "combine_int<typename Ctx::ISum>" in code and "splat_int<kVec>" in code


def test_pointwise_uses_128bit_access_when_contiguous(dry_backend):
    code = generated(lambda a, b: F.silu(a) * b, torch.randn(8, 1000).bfloat16(), torch.randn(8, 1000).bfloat16())
    assert "launch_pointwise<Body>" in code and "kVec = 8" in code
    # unconditional 128-bit access in full tiles: the flat index is a multiple of the vector
    assert code.count("ldvec<ixb::bf16, kVec, FAST>") == 2 and "stvec<ixb::bf16, kVec, FAST>" in code
    assert "pointers_aligned(ptrs, 3)" in code
    assert "gather(" not in code


def test_permuted_store_falls_back_to_scatter_or_gather(dry_backend):
    code = generated(lambda t: (t.permute(0, 2, 1) + 1).contiguous(), torch.randn(4, 16, 24))
    assert "launch_pointwise<Body>" in code
    assert "gather(" in code or "scatter(" in code


def test_transpose_is_staged_as_register_tiles(dry_backend):
    """Loads contiguous along another digit of the flat index than the stores: 128-bit loads of
    a V x kC micro-tile per thread, kC 128-bit stores, lanes 4 x 8."""
    code = generated(lambda t: (t.permute(0, 1, 3, 2) * 2).contiguous(), torch.randn(8, 8, 512, 128).half())
    assert "launch_pointwise_tile<Body>" in code
    assert "static constexpr int kTileC = 8;" in code and "static constexpr long long kStepC = 512LL;" in code
    assert "ixb::gen::fetch_tile(raw.t0, in_ptr0," in code and "STAGED ? ixb::gen::take(raw.t0, ci)" in code
    assert "stvec<ixb::f16, kVec, FAST>" in code
    # an innermost-preserving permute needs none of it: vector access on both sides
    code = generated(lambda t: (t.permute(0, 2, 1, 3) + 1).contiguous(), torch.randn(8, 8, 512, 128).half())
    assert "launch_pointwise<Body>" in code and "gather(" not in code


def test_strided_reduction_over_contiguous_outputs_uses_outer_mapping(dry_backend):
    """Reduced axes are not innermost (reference case test_reduction_permute): adjacent
    threads must walk adjacent outputs, not the strided reduction axis."""
    x = torch.randn(4, 8, 16, 64).half()
    code = generated(lambda t: t.permute(0, 3, 1, 2).amax((2, 3)), x)
    assert code.count("ixb_load_kernel('''") == 1
    # 64 contiguous fp16 outputs = 8 vectors: 8 threads along the kept axis, the rest of
    # each warp walks the reduced axis
    assert "launch_outer_gen<Body, 8>" in code and "family='outer'" in code
    assert "c.template combine<ixb::MaxOp>(acc)" in code
    # full aligned tiles issue the loads of eight reduced steps as raw 128-bit words and pin
    # them before the first is widened; ragged tiles keep the plain loop
    assert "if constexpr (FAST)" in code and "RawVec<ixb::f16, kVec> raw_tmp0[8];" in code
    assert "ixb::gen::ldraw<ixb::f16, kVec>(" in code and "ixb::gen::pin(raw_tmp0[u]);" in code
    assert "ixb::gen::widen_raw(raw_tmp0[u])" in code
    # an inner-axis reduction of the same tensor keeps the row mapping
    code = generated(lambda t: t.amax(-1), x)
    assert "launch_row_gen<" in code and "launch_outer_gen" not in code


def test_long_rows_are_walked_in_chunks(dry_backend):
    # rows beyond MAX_TEAM x MAX_PERSISTENT_VPT vectors: one chunk loop per dependent reduction,
    # accumulators ahead of the loop, one team exchange after it
    code = generated(lambda t: torch.log_softmax(t, -1), torch.randn(4, 128256))
    assert code.count("ixb_load_kernel('''") == 1
    assert code.count("for (int chunk = 0; chunk < c.nchunks(); ++chunk)") == 2
    assert "c.online_chunk(_acc0," in code and "c.online_finish(_acc0)" in code
    assert "static constexpr bool kLooped = true;" in code and "tune=dict(" not in code
    code = generated(lambda t: torch.var_mean(t, -1), torch.randn(4, 300000))
    assert "c.local_welford(" in code or code.count("c.nchunks()") == 2
    # a row that fits stays on chip
    code = generated(lambda t: torch.log_softmax(t, -1), torch.randn(4, 32768))
    assert "c.nchunks()" not in code and "static constexpr bool kLooped = false;" in code


def test_index_analysis_is_structural():
    """Which addresses a kernel reads is decided from the form of the index, not from
    sample points: mixed-radix digits of the reduced index must tile its range."""
    from inductor_x_b200.codegen import ir
    from torch.utils._sympy.functions import FloorDiv, ModularIndexing

    x, r = sympy.Symbol("xindex", integer=True, nonnegative=True), sympy.Symbol("r0_index", integer=True, nonnegative=True)
    assert ir.reduction_stride(ModularIndexing(r, 1, 8) + 8 * FloorDiv(r, 8), x, r, 4, 64) == 1
    assert ir.reduction_stride(ModularIndexing(r, 1, 8) + 8 * ModularIndexing(r, 8, 8) + 64 * x, x, r, 4, 64) == 1
    assert ir.reduction_stride(ModularIndexing(r, 1, 8) + 8 * ModularIndexing(r, 8, 4) + 64 * x, x, r, 4, 64) is None
    assert ir.reduction_stride(2 * ModularIndexing(r, 1, 8) + 16 * ModularIndexing(r, 8, 8) + x, x, r, 4, 64) == 2
    assert ir.reduction_stride(ModularIndexing(x + r, 1, 8), x, r, 4, 64) is None
    assert ir.row_starts_aligned(r + 4096 * x, x, r, 8) and not ir.row_starts_aligned(r + 1023 * x, x, r, 8)
    assert ir.x_contiguous_for_all_r(ModularIndexing(x, 1, 64) + 64 * r + 16384 * FloorDiv(x, 64), x, r, 8)
    assert not ir.x_contiguous_for_all_r(64 * ModularIndexing(x, 1, 64) + r, x, r, 8)


def test_index_analysis():
    from inductor_x_b200.codegen import ir
    from torch.utils._sympy.functions import FloorDiv, ModularIndexing

    x, r = sympy.Symbol("xindex", integer=True, nonnegative=True), sympy.Symbol("r0_index", integer=True, nonnegative=True)
    # flat contiguous and row-broadcast accesses are vector-contiguous, a transpose is not
    assert ir.is_vector_contiguous(x, x, 8, 1 << 20)
    assert ir.is_vector_contiguous(ModularIndexing(x, 1, 4096), x, 8, 1 << 20)
    assert ir.is_vector_contiguous(ModularIndexing(x, 1, 4096) + 4096 * FloorDiv(x, 4096), x, 8, 1 << 20)
    assert not ir.is_vector_contiguous(64 * ModularIndexing(x, 1, 128) + FloorDiv(x, 128), x, 8, 1 << 13)
    assert not ir.is_vector_contiguous(ModularIndexing(x, 1, 1023), x, 8, 1023 * 8)
    # reduction strides: inner (1), outer (constant > 1), flattened multi-axis (None)
    assert ir.reduction_stride(r + 4096 * x, x, r, 100, 4096) == 1
    assert ir.reduction_stride(ModularIndexing(x, 1, 64) + 64 * r + 16384 * FloorDiv(x, 64), x, r, 8192, 256) == 64
    assert ir.reduction_stride(x, x, r, 10, 10) == 0
    assert ir.reduction_stride(ModularIndexing(r, 1, 8) * 100 + FloorDiv(r, 8), x, r, 4, 64) is None


def test_launch_chooser():
    from inductor_x_b200.codegen import split_tiling as st

    c = st.choose_row_config(4096, torch.bfloat16, rows=16384)
    assert (c.team, c.vpt, c.vec, c.teams, c.min_ctas, c.prefetch) == (256, 2, 8, 1, 4, 2)
    assert st.choose_row_config(4096, torch.bfloat16, rows=32).prefetch == 0    # nothing to stream
    c = st.choose_row_config(1000, torch.float32)
    assert c.capacity >= 1000 and c.vec == 4 and (c.team, c.vpt) == (128, 2)
    c = st.choose_row_config(64, torch.float16)                      # 8 vectors: a quarter warp per row
    assert (c.team, c.vpt, c.teams) == (8, 1, 16)
    c = st.choose_row_config(32768, torch.float32)                   # beyond 1024 x 2 vectors
    assert (c.team, c.vpt) == (1024, 8)
    c = st.choose_row_config(128256, torch.float32)                  # a vocabulary-sized fp32 row: spills, but runs
    assert (c.team, c.vpt) == (1024, 32)
    assert st.choose_row_config(1 << 20, torch.float32) is None
    assert st.choose_pointwise_vec([torch.float32, torch.bfloat16]) == 8
    assert st.choose_pointwise_vec([torch.float32]) == 4
    assert st.should_use_persistent_reduction(4096, torch.bfloat16)
    assert not st.should_use_persistent_reduction(sympy.Symbol("s0"), torch.float32)


def test_registration_surface():
    import inductor_x_b200
    from inductor_x_b200 import decomposition, fusion_attention_graph, lowering
    from torch._inductor.codegen.common import get_scheduling_for_device

    assert get_scheduling_for_device("cuda").__name__ == "B200Scheduling"
    assert callable(inductor_x_b200.get_current_raw_stream)
    assert all(present for _, present in decomposition._register_b200_inductor_decompositions())
    s = set()
    lowering._init_set([torch.ops.aten.cumsum], s)
    assert torch.ops.aten.cumsum.default in s
    assert hasattr(torch.ops.b200_graph, "b200_fa") and hasattr(torch.ops.b200_graph, "b200_fa_backward")
    # Meta implementation mirrors the reference's output shapes (softmax stats [B, N, S, 8])
    q = torch.empty(2, 4, 16, 128, device="meta", dtype=torch.bfloat16)
    out = torch.ops.b200_graph.b200_fa(q, q, q, 4, "BNSD")
    assert out[0].shape == q.shape and out[1].shape == (2, 4, 16, 8) and len(out) == 7


def test_short_rows_of_a_whole_line_walk_the_output_digit_first(dry_backend):
    """Config 3a's sum: rows of 128 bytes that are far apart along the output's fastest digit.
    The kept index is walked in 16 x 16 tiles with the OUTPUT digit fastest inside a tile (the
    sixteen rows a warp works on store one 32-byte sector); rows shorter than a line keep the
    input-contiguous order."""
    x = torch.randn(4, 32, 64, 64).half()
    code = generated(lambda t: t.permute(0, 2, 1, 3).sum(3), x)
    assert "ixb::gen::tile_order<32, 64, 16, 16, true>(xslot)" in code
    x = torch.randn(4, 32, 64, 16).half()
    code = generated(lambda t: t.permute(0, 2, 1, 3).sum(3), x)
    assert "tile_order<32, 64, 16, 16, false>(xslot)" in code


def test_cumsum_over_the_last_axis_is_scanned_by_the_row_template(dry_backend):
    """A floating cumsum along the stride-1 axis becomes a row kernel with a team-wide prefix
    sum (fused with the pointwise work around it); other axes and other output dtypes stay extern
    kernels, which is all the reference does for cumsum (inductor_x/lowering.py:235-245)."""
    x = torch.randn(64, 1024)
    code = generated(lambda t: torch.cumsum(t * 2.0, -1) + 1.0, x)
    assert code.count("ixb_load_kernel('''") == 1 and "c.template scan<ixb::SumOp>(" in code and "launch_row_gen<" in code
    extern = "torch.ops.aten.cumsum.default("
    assert extern not in code
    code = generated(lambda t: torch.cumsum(t, 0), x)
    assert "c.template scan<" not in code and extern in code
    # integer rows are summed exactly in 64 bits
    code = generated(lambda t: torch.cumsum(t, -1), torch.arange(64 * 128).reshape(64, 128))
    assert "c.template scan_int<typename Ctx::ISum>(" in code and extern not in code
    code = generated(lambda t: torch.cumsum(t, -1, dtype=torch.float64), x)
    assert "c.template scan" not in code and extern in code
    # cumprod takes the same path with the product operator; cummax stays extern
    code = generated(lambda t: torch.cumprod(t, -1), x)
    assert "c.template scan<ixb::ProdOp>(" in code and "torch.ops.aten.cumprod.default(" not in code
    code = generated(lambda t: torch.cummax(t, -1)[0], x)
    assert "c.template scan" not in code and "torch.ops.aten.cummax.default(" in code


def test_long_scans_of_few_rows_are_never_cut_into_split_scans(dry_backend, monkeypatch):
    """Inductor's split heuristic would cut a long scan with few kept rows in two (a decoupled
    look-back kernel, which only its Triton backend writes); on this backend the row template
    holds the whole row, so the node stays a plain Scan that fuses like any reduction."""
    from torch._inductor import ir as inductor_ir

    made = []
    stock = inductor_ir.SplitScan.__init__

    def spy(self, *a, **k):
        made.append(1)
        return stock(self, *a, **k)

    monkeypatch.setattr(inductor_ir.SplitScan, "__init__", spy)
    for shape in ((1, 16384), (16384,), (2, 16384), (4, 12000)):
        code = generated(lambda t: torch.cumsum(t, -1).sum(-1), torch.randn(*shape))
        assert "c.template scan<ixb::SumOp>(" in code and "triton_" not in code
        assert code.count("ixb_load_kernel(" + "'" * 3) == 1     # the scan and the sum after it: one kernel
    assert not made


def test_integer_bitwise_ops_keep_the_bit_pattern(dry_backend):
    """and / or / xor / not print as bit operations for integer operands and as logical ones
    for booleans; shifts exist; a left shift and the complement of an unsigned byte are wrapped
    back into the range of their type (integers are carried in 64 bits)."""
    a, b = torch.randint(1, 100, (1000,)), torch.randint(0, 5, (1000,))
    code = generated(lambda a, b: ((a & b) | (a ^ 7)) + (~a) + (a << b) + (a >> b), a, b)
    for name in ("bit_and(", "bit_or(", "bit_xor(", "bit_not(", "lshift(", "rshift("):
        assert "ixb::gen::op::" + name in code
    assert "logical_" not in code and "wrap_int" not in code        # 64-bit values need no wrap
    code = generated(lambda a, b: (a > 3) & (b < 2) | ~(a == b), a, b)
    assert "logical_and(" in code and "logical_not(" in code and "bit_" not in code
    code = generated(lambda a, b: (a.to(torch.int32) << b.to(torch.int32)) + 1, a, b)
    assert "wrap_int<32, true>(ixb::gen::op::lshift(" in code
    code = generated(lambda a: (~a).float(), a.to(torch.uint8))
    assert "wrap_int<8, false>(ixb::gen::op::bit_not(" in code


def test_narrowing_integer_conversions_wrap(dry_backend):
    """int64 -> int8 / uint8 / int16 / int32 wraps like the stored value would, and so do sums,
    differences and products of integers narrower than 64 bits; widening conversions and
    conversions from floating values are plain."""
    a = torch.randint(-1000, 1000, (1000,))
    code = generated(lambda a: a.to(torch.uint8).float() + a.to(torch.int8).float(), a)
    assert "wrap_int<8, false>(" in code and "wrap_int<8, true>(" in code
    code = generated(lambda a: a.to(torch.int64) * 3, a.to(torch.int32))
    assert "wrap_int" not in code
    code = generated(lambda x: (x * 10).to(torch.int32) + 1, torch.randn(1000))
    assert "(ixb::gen::op::to_int(" not in code                    # the conversion itself is plain ...
    assert "wrap_int<32, true>(ixb::gen::op::add(" in code         # ... the int32 sum after it can overflow


def test_ops_without_a_template_stay_extern_and_the_rest_compiles(dry_backend):
    """Random numbers come from ATen's generators (dropout in training mode compiles, the scaling
    around it is generated); scans with other operators and the special functions Inductor only
    has in its own backends stay extern kernels; inverse hyperbolic functions, erfinv, ldexp and
    nextafter are generated; a constant pad (a masked sub-block) is generated."""
    x = torch.rand(64, 256) * 0.8 + 0.1
    code = generated(lambda t: F.dropout(t * 2.0, 0.1, True) + 1.0, x)
    assert "ixb_load_kernel(" in code and ("aten.native_dropout" in code or "aten.bernoulli" in code
                                           or "aten.rand" in code)
    code = generated(lambda t: torch.logcumsumexp(t, -1), x)
    assert "torch.ops.aten.logcumsumexp.default(" in code and "c.template scan" not in code
    code = generated(lambda t: torch.digamma(t) + torch.special.i0(t), x)
    assert "torch.ops.aten.digamma.default(" in code and "torch.ops.aten.i0.default(" in code
    code = generated(lambda t: torch.asinh(t) + torch.acosh(t + 1) + torch.atanh(t) + torch.erfinv(t)
                     + torch.nextafter(t, t + 1) + torch.ldexp(t, torch.tensor(3)), x)
    for name in ("asinh(", "acosh(", "atanh(", "erfinv(", "nextafter("):
        assert "ixb::gen::op::" + name in code
    assert code.count("ixb_load_kernel(") == 1
    code = generated(lambda t: F.max_pool2d(F.pad(t, (1, 2, 3, 4), value=-1.0), 3, 2, 1), torch.randn(2, 3, 16, 16))
    assert code.count("ixb_load_kernel(") == 1 and "= torch.ops.aten.constant_pad_nd.default(" not in code
    assert "ixb::gen::op::where(" in code                 # the pad value outside the source's bounds


def test_a_library_transformer_compiles_through_the_templates(dry_backend):
    """A small DistilBERT from the transformers library (random weights, dropout active) compiles
    with every fused group instantiated from the templates: no Triton kernel, no refusal from the
    emitter, the dropout masks drawn by ATen's generator."""
    transformers = pytest.importorskip("transformers")
    cfg = transformers.DistilBertConfig(dim=128, n_layers=1, n_heads=4, hidden_dim=256, vocab_size=1000)
    model = transformers.DistilBertModel(cfg).train()
    ids = torch.randint(0, 1000, (2, 32))
    with torch.no_grad():
        code = generated(lambda input_ids: model(input_ids=input_ids)[0], ids)
    assert code.count("ixb_load_kernel(") >= 4 and "triton_" not in code
    assert "aten.native_dropout" in code or "aten.bernoulli" in code or "aten.rand" in code


def test_integer_arg_reductions_compare_integers(dry_backend):
    """argmax / argmin of int32 / int64 rows use the integer comparison (persistent and chunked
    rows); narrower integers are exact in fp32 and keep the common path."""
    big = (torch.arange(64 * 300).reshape(64, 300) % 7) + (1 << 40)
    code = generated(lambda t: (t.argmax(-1), t.argmin(-1)), big)
    assert "c.template reduce_arg_int<true>(" in code and "c.template reduce_arg_int<false>(" in code
    code = generated(lambda t: t.argmax(-1), torch.randint(0, 1 << 40, (4, 70000)))
    assert "c.template local_arg_int<true>(" in code and "c.template xreduce_arg_int<true>(" in code
    code = generated(lambda t: t.argmin(-1), big.to(torch.uint8))
    assert "c.template reduce_arg<false>(" in code


def test_symbolic_extents_print_python_mod_and_true_division(dry_backend):
    """Forms that only appear with run-time extents: Python's modulo (a rolled index) and the
    true division of two extents (the n / (n - 1) factor of a batch-norm's running variance)."""
    import torch._dynamo

    def compiled_dynamic(fn, *args):
        from torch._inductor.utils import run_and_get_code

        torch._dynamo.reset()
        _, code = run_and_get_code(torch.compile(fn, dynamic=True), *args)
        return "\n".join(code)

    code = compiled_dynamic(lambda t: t.roll(3, -1) + 1, torch.randn(4, 64))
    assert "ixb::gen::op::remainder(" in code and "ixb_load_kernel(" in code
    bn = torch.nn.BatchNorm2d(16).train()
    code = compiled_dynamic(bn, torch.randn(8, 16, 14, 14))
    assert "ixb::gen::op::truediv(ixb::gen::op::to_float(" in code and "triton_" not in code
    # a non-finite pad value behind an integer load (max-pooling integers converted to float)
    code = generated(lambda a: F.max_pool1d(a.view(1, 1, 100).float(), 3, 1, 1), torch.randint(1, 10, (100,)))
    assert "ixb_load_kernel(" in code


def test_long_rows_of_run_time_length_are_walked_in_chunks(dry_backend):
    """A symbolic reduced extent whose trace-time value is beyond every launch shape (a full
    reduction of a tensor with run-time sizes, a very long softmax row) becomes the chunked row
    kernel: the chunk count comes from the extent the launcher passes, so any length is served."""
    from torch._inductor.utils import run_and_get_code

    for fn, x in ((lambda t: t.sum(), torch.randn(1000, 1000)), (lambda t: t.softmax(-1), torch.randn(4, 200000))):
        torch._dynamo.reset()
        _, code = run_and_get_code(torch.compile(fn, dynamic=True), x)
        code = "\n".join(code)
        assert "static constexpr bool kLooped = true;" in code and "c.nchunks()" in code
        assert "long long r_extent;" in code and "(int)r_extent" in code


def test_python_float_arguments_are_baked_into_the_graph(dry_backend):
    """With dynamic shapes a Python float would enter the graph as a 0-dim float64 host tensor;
    registration specialises floats instead, so the scale is a literal of the generated kernel."""
    from torch._inductor.utils import run_and_get_code

    torch._dynamo.reset()
    _, code = run_and_get_code(torch.compile(lambda t, s: t * s + 1, dynamic=True), torch.randn(64, 100), 0.37)
    code = "\n".join(code)
    assert "0.37f" in code and "double" not in code.split("extern \"C\"")[0].split("struct Body")[1]


def test_integer_range_helpers():
    """Host logic behind the integer wrap: which conversions can leave the target's range and
    how a wrap is printed."""
    import inductor_x_b200  # noqa: F401
    from inductor_x_b200.codegen.overrides import _fits, _narrow_int_result, _wrap

    assert _fits(torch.uint8, torch.int16) and _fits(torch.int8, torch.int32) and _fits(torch.bool, torch.uint8)
    assert _fits(torch.int32, torch.int64) and _fits(torch.int16, torch.int16)
    assert not _fits(torch.int64, torch.int32) and not _fits(torch.int8, torch.uint8)      # sign is lost
    assert not _fits(torch.uint8, torch.int8) and not _fits(torch.float32, torch.int64)
    assert _wrap("v", torch.int64) == "v" and _wrap("v", torch.bool) == "v" and _wrap("v", None) == "v"
    assert _wrap("v", torch.uint8) == "ixb::gen::op::wrap_int<8, false>(v)"
    assert _wrap("v", torch.int16) == "ixb::gen::op::wrap_int<16, true>(v)"

    class Val:
        def __init__(self, dtype, int_type=None):
            self.dtype, self.int_type = dtype, int_type

    i32, u8, i64 = Val(torch.int64, torch.int32), Val(torch.int64, torch.uint8), Val(torch.int64)
    assert _narrow_int_result(i32, 3) == torch.int32                 # Python scalars do not promote
    assert _narrow_int_result(i32, u8) == torch.int32 and _narrow_int_result(u8, Val(torch.bool)) == torch.uint8
    assert _narrow_int_result(i32, i64) is None                      # 64-bit results need no wrap
    assert _narrow_int_result(i32, Val(torch.float32)) is None       # not an integer result
