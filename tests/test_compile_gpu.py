"""GPU tests of the torch.compile path: graphs compiled through the B200 backend (template
instantiation, no Triton) against eager PyTorch on the same inputs - the discipline of the
reference's own tests (test/npu_indexing/reduction_test.py:28-30, permute_test.py:24-29),
with the tolerances of this build: rel 1e-5 fp32 reductions, 2e-2 half, bit-exact indices."""
import pytest
import torch
import torch.nn.functional as F

import inductor_x_b200  # noqa: F401  (registers the backend for "cuda")
from oracle import graphs, inputs

pytestmark = pytest.mark.gpu


def compile_and_code(fn, *args):
    from torch._inductor.utils import run_and_get_code

    torch._dynamo.reset()
    out, code = run_and_get_code(torch.compile(fn), *args)
    text = "\n".join(code)
    # no Triton kernel anywhere in the generated module: every fused group is a template instantiation
    assert "triton_" not in text.replace("triton_helpers", "").replace("triton_heuristics", "")
    return out, text


def test_c1_one_fused_kernel(cuda):
    d = inputs.c1(512, 1024, seed=3)
    x, w, b = (d[k].to(cuda) for k in ("x", "w", "b"))
    out, code = compile_and_code(lambda x, w, b: F.gelu(x * w + b).sum(-1), x, w, b)
    assert code.count("ixb_load_kernel('''") == 1  # the reference needs three kernels here
    assert graphs.max_rel_err(out.cpu(), graphs.affine_gelu_rowsum(d["x"].double(), d["w"].double(), d["b"].double())) <= 1e-5


def test_c2_one_fused_kernel(cuda):
    d = inputs.c2(256, 4096, seed=4)
    x, g, ga, be = (d[k].to(cuda) for k in ("x", "g", "gamma", "beta"))
    fn = lambda x, g, ga, be: F.layer_norm(torch.softmax(x, -1) * g + x, (4096,), ga, be, 1e-5)
    out, code = compile_and_code(fn, x, g, ga, be)
    assert code.count("ixb_load_kernel('''") == 1
    exp = graphs.softmax_layernorm(**d, compute=torch.float64, round_output=False)
    assert graphs.max_rel_err(out.cpu(), exp) <= 2e-2


@pytest.mark.parametrize("shape", [(8, 32, 512, 64), (8, 8, 512, 128), (2053, 1023), (513, 64), (3, 7, 9)])
def test_pointwise_shapes(cuda, shape):
    g = torch.Generator().manual_seed(sum(shape))
    a = torch.randn(*shape, generator=g).to(cuda)
    b = torch.randn(*shape, generator=g).to(cuda)
    fn = lambda a, b: torch.sigmoid(a) * b + torch.relu(a - b) * 0.5
    out, _ = compile_and_code(fn, a, b)
    torch.testing.assert_close(out, fn(a, b), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,dim", [((8, 16, 512, 64), -1), ((8, 16, 512, 64), 2), ((8, 16, 512, 64), 1),
                                       ((8, 16, 512, 64), 0), ((2053, 1023), -1), ((64, 1000), 1),
                                       ((37, 4096), 1)])
def test_sum_mean_dims(cuda, dtype, shape, dim):
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(*shape, generator=g).to(dtype).to(cuda)
    for op in (torch.sum, torch.mean, torch.amax):
        out, _ = compile_and_code(lambda t: op(t, dim), x)
        exp = op(x.double(), dim)
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        floor = float(exp.abs().mean()) or 1.0
        assert graphs.max_rel_err(out.cpu(), exp.cpu(), floor=floor) <= tol


@pytest.mark.parametrize("perm", [(0, 2, 1, 3), (3, 2, 1, 0), (0, 1, 3, 2), (1, 0, 2, 3)])
def test_permute_pointwise(cuda, perm):
    x = torch.randn(8, 8, 64, 128, generator=torch.Generator().manual_seed(1)).to(cuda)
    fn = lambda t: (t.permute(*perm) + 1.0).contiguous()
    out, _ = compile_and_code(fn, x)
    assert torch.equal(out, fn(x))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape,perm,tiled", [((4, 8, 512, 128), (0, 1, 3, 2), True), ((6, 256, 512), (0, 2, 1), True),
                                              ((8, 8, 64, 128), (3, 2, 1, 0), False), ((3, 40, 72), (0, 2, 1), False)])
def test_transposes_use_register_tiles(cuda, dtype, shape, perm, tiled):
    """A pointwise group that stores along the flat index and reads along another digit of it:
    every thread loads a V x kC micro-tile with 128-bit loads and stores kC 128-bit vectors
    (where the extents allow; the last two shapes do not and keep per-element gathers).
    Copies must be bit-exact."""
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(*shape, generator=g).to(dtype).to(cuda)
    fn = lambda t: (t.permute(*perm) * 2.0).contiguous()
    out, code = compile_and_code(fn, x)
    assert torch.equal(out, fn(x))
    assert ("launch_pointwise_tile<Body>" in code and "take(raw.t0, ci)" in code) == tiled
    # a second operand in the output's layout rides along as an ordinary vector load
    y = torch.randn(*out.shape, generator=g).to(dtype).to(cuda)
    fn2 = lambda t, u: (t.permute(*perm) + u).contiguous()
    out2, _ = compile_and_code(fn2, x, y)
    assert torch.equal(out2, fn2(x, y))
    # a misaligned base pointer takes the plain kernel of the same module
    xo = torch.randn(x.numel() + 1, generator=g).to(dtype).to(cuda)[1:].view(*shape)
    out3, _ = compile_and_code(fn, xo)
    assert torch.equal(out3, fn(xo))


def test_c3a_permuted_reductions(cuda):
    x = inputs.c3a((8, 16, 64, 64), seed=2)["x"].to(cuda)
    amax, _ = compile_and_code(lambda t: t.permute(0, 2, 1, 3).amax(1), x)
    assert torch.equal(amax, x.permute(0, 2, 1, 3).amax(1))
    ssum, _ = compile_and_code(lambda t: t.permute(0, 2, 1, 3).sum(3), x)
    assert graphs.max_rel_err(ssum.cpu(), graphs.permuted_sum(x.cpu(), torch.float64)) <= 2e-2


def test_var_mean_and_argmax(cuda):
    x = torch.randn(64, 1000, generator=torch.Generator().manual_seed(5)).to(cuda)
    (var, mean), _ = compile_and_code(lambda t: torch.var_mean(t, -1), x)
    ev, em = torch.var_mean(x.double(), -1)
    assert graphs.max_rel_err(var.cpu(), ev.cpu()) <= 1e-5
    assert graphs.max_rel_err(mean.cpu(), em.cpu(), floor=0.05) <= 1e-5
    idx, _ = compile_and_code(lambda t: torch.argmax(t, -1), x)
    assert torch.equal(idx, torch.argmax(x, -1))


def test_index_select_and_embedding(cuda):
    d = inputs.c3b(4096, 128, 2048, seed=6)
    table, idx = d["table"].to(cuda), d["idx"].to(cuda)
    out, code = compile_and_code(lambda t, i: t.index_select(0, i) * 1, table, idx)
    assert "ixb_load_kernel" in code
    assert torch.equal(out, table.index_select(0, idx))


def test_rmsnorm_swiglu_rope(cuda):
    g = torch.Generator().manual_seed(8)
    x = torch.randn(64, 4096, generator=g).bfloat16().to(cuda)
    w = (1 + 0.1 * torch.randn(4096, generator=g)).bfloat16().to(cuda)
    rms = lambda x, w: (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(x.dtype) * w
    out, code = compile_and_code(rms, x, w)
    assert code.count("ixb_load_kernel('''") == 1
    assert graphs.max_rel_err(out.cpu(), graphs.rmsnorm(x.cpu(), w.cpu(), 1e-6, torch.float64)) <= 2e-2
    up = torch.randn(64, 4096, generator=g).bfloat16().to(cuda)
    out, _ = compile_and_code(lambda a, b: F.silu(a) * b, x, up)
    assert graphs.max_rel_err(out.cpu(), graphs.swiglu(x.cpu(), up.cpu(), torch.float64)) <= 2e-2
    q = torch.randn(2, 4, 64, 128, generator=g).bfloat16().to(cuda)
    cos, sin = (t.to(cuda) for t in inputs.rope_tables(64, 128))

    def rope(q, cos, sin):
        d = q.shape[-1] // 2
        rot = torch.cat([-q[..., d:], q[..., :d]], -1)
        return (q.float() * cos + rot.float() * sin).to(q.dtype)

    out, _ = compile_and_code(rope, q, cos, sin)
    assert graphs.max_rel_err(out.cpu(), graphs.rope(q.cpu(), cos.cpu(), sin.cpu(), torch.float64)) <= 2e-2


def test_sdpa_is_retargeted_to_the_tcgen05_kernel(cuda):
    d = inputs.c4(2, 4, 512, 128, seed=9)
    q, k, v = (d[n].to(cuda) for n in "qkv")
    fn = lambda q, k, v: F.scaled_dot_product_attention(q, k, v, is_causal=True)
    out, code = compile_and_code(fn, q, k, v)
    assert "b200_sdpa" in code
    exp, _ = graphs.attention(d["q"], d["k"], d["v"], d["scale"], causal=True)
    assert graphs.max_rel_err(out.cpu(), exp, dim=-1) <= 2e-2


def test_reference_attention_pattern_is_matched(cuda):
    from inductor_x_b200 import config

    p = inputs.c4_pattern(2, 128, 4, 128, seed=4)
    inv = p["inv_scale_factor"]

    def pattern(query, key, value):
        qq, kk, vv = (t.permute(0, 2, 1, 3) for t in (query, key, value))
        return torch.matmul(qq, kk.transpose(-2, -1)).div(inv).softmax(dim=-1).matmul(vv)

    exp = graphs.attention_pattern(p["query"], p["key"], p["value"], inv)
    # 16-bit operands: matched and run on the tcgen05 kernel (expected values from the same
    # rounded operands)
    q, k, v = (p[n].bfloat16().to(cuda) for n in ("query", "key", "value"))
    out, code = compile_and_code(pattern, q, k, v)
    assert "b200_fa" in code
    exp16 = graphs.attention_pattern(q.float().cpu(), k.float().cpu(), v.float().cpu(), inv)
    assert graphs.max_rel_err(out.float().cpu(), exp16, dim=-1) <= 2e-2
    # float32 operands (what the reference traces its pattern with): narrowing them to
    # fp16 is the caller's choice - left alone by default, matched with the opt-in
    q, k, v = (p[n].to(cuda) for n in ("query", "key", "value"))
    out, code = compile_and_code(pattern, q, k, v)
    assert "b200_fa" not in code
    assert graphs.max_rel_err(out.cpu(), exp, dim=-1) <= 1e-4
    config.attention_fp32_as_fp16 = True
    try:
        out, code = compile_and_code(pattern, q, k, v)
    finally:
        config.attention_fp32_as_fp16 = False
    assert "b200_fa" in code
    assert graphs.max_rel_err(out.cpu(), exp, dim=-1) <= 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_literal_causal_attention_graph_runs_on_the_tcgen05_kernel(cuda, dtype):
    """Benchmark configuration 4 as it is written - matmul, scale, masked_fill with a causal
    mask built in the graph, softmax, matmul - at reduced batch and sequence length."""
    d = inputs.c4(2, 4, 512, 128, seed=12)
    q, k, v = (d[n].to(dtype).to(cuda) for n in "qkv")
    scale = d["scale"]

    def attention(q, k, v):
        n = q.shape[-2]
        keep = torch.ones(n, n, dtype=torch.bool, device=q.device).tril()
        s = torch.matmul(q, k.transpose(-2, -1)) * scale
        s = s.masked_fill(~keep, float("-inf"))
        return torch.matmul(torch.softmax(s, dim=-1), v)

    out, code = compile_and_code(attention, q, k, v)
    assert "b200_sdpa" in code and "bmm" not in code
    exp, _ = graphs.attention(q.cpu(), k.cpu(), v.cpu(), scale, causal=True)
    assert graphs.max_rel_err(out.cpu(), exp, dim=-1) <= 2e-2


def test_causal_sdpa_with_longer_keys_is_left_to_aten(cuda):
    """torch masks is_causal from the top-left corner; the kernel's causal mode is aligned
    bottom-right.  They differ when Sk > Sq, so such a node must not be retargeted."""
    g = torch.Generator().manual_seed(17)
    q = torch.randn(2, 4, 128, 128, generator=g).bfloat16().to(cuda)
    k, v = (torch.randn(2, 4, 256, 128, generator=g).bfloat16().to(cuda) for _ in range(2))
    fn = lambda q, k, v: F.scaled_dot_product_attention(q, k, v, is_causal=True)
    out, code = compile_and_code(fn, q, k, v)
    assert "b200_sdpa" not in code
    want = F.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=True)
    assert graphs.max_rel_err(out.float().cpu(), want.cpu(), dim=-1) <= 2e-2
    # grouped-query shapes (fewer key/value heads) are not the kernel's either
    k2, v2 = (torch.randn(2, 1, 128, 128, generator=g).bfloat16().to(cuda) for _ in range(2))
    fn2 = lambda q, k, v: F.scaled_dot_product_attention(q, k, v, enable_gqa=True)
    out, code = compile_and_code(fn2, q, k2, v2)
    assert "b200_sdpa" not in code


def test_integer_reductions_are_exact(cuda):
    """Integer sums and extrema run on 64-bit accumulators and exchanges: values beyond
    2^24 (where an fp32 path would round) come out bit-exact, along rows and along columns."""
    g = torch.Generator().manual_seed(23)
    ids = torch.randint(0, 1 << 40, (257, 4096), generator=g).to(cuda)
    (s, m, c), code = compile_and_code(lambda t: (t.sum(-1), t.amax(-1), t.sum(0)), ids)
    assert "reduce_int<" in code and "combine_int<" in code
    assert torch.equal(s, ids.sum(-1)) and torch.equal(m, ids.amax(-1)) and torch.equal(c, ids.sum(0))
    ones = torch.ones(1 << 25, 2, dtype=torch.int32, device=cuda)      # 2^25 ones per column
    s, _ = compile_and_code(lambda t: t.sum(0), ones)
    assert s.tolist() == [1 << 25] * 2
    big = torch.full((5, 1 << 17), 1 << 12, dtype=torch.int32, device=cuda)   # row sums of 2^29
    s, _ = compile_and_code(lambda t: t.sum(-1, dtype=torch.int64), big)
    assert s.tolist() == [1 << 29] * 5
    mask = (torch.rand(64, 5000, generator=g) > 0.5).to(cuda)
    cnt, _ = compile_and_code(lambda t: t.sum(-1), mask)
    assert torch.equal(cnt, mask.sum(-1))


def test_dynamic_row_counts_share_one_module(cuda):
    """torch.compile(dynamic=True): the kept extent reaches the launcher at run time (the
    reference passes symbolic numel arguments the same way, inductor_x/codegen/wrapper.py:21-38),
    so three row counts of the C1 and C2 graphs run on one generated module each."""
    from inductor_x_b200.codegen import jit

    c2 = lambda x, g, ga, be: F.layer_norm(torch.softmax(x, -1) * g + x, (4096,), ga, be, 1e-5)
    c1 = lambda x, w, b: F.gelu(x * w + b).sum(-1)
    for graph, make, ref, tol in (
            (c2, lambda r: inputs.c2(r, 4096, seed=r), lambda d: graphs.softmax_layernorm(**d, compute=torch.float64, round_output=False), 2e-2),
            (c1, lambda r: inputs.c1(r, 1024, seed=r), lambda d: graphs.affine_gelu_rowsum(d["x"].double(), d["w"].double(), d["b"].double()), 1e-5)):
        torch._dynamo.reset()
        fn = torch.compile(graph, dynamic=True)
        modules = None
        for rows in (96, 257, 1000):
            d = make(rows)
            out = fn(*(v.to(cuda) for v in d.values() if isinstance(v, torch.Tensor)))
            assert out.shape[0] == rows
            assert graphs.max_rel_err(out.cpu(), ref(d)) <= tol
            if modules is None:
                modules = len(jit._loaded)
            assert len(jit._loaded) == modules          # no new module for a new row count


def test_dynamic_reduced_extent_within_compiled_capacity(cuda):
    """A symbolic reduced extent is served up to the capacity of the launch shape compiled for
    the first extent; a longer row is refused by the launcher, never mis-computed."""
    torch._dynamo.reset()
    fn = torch.compile(lambda t: torch.softmax(t, -1), dynamic=True)
    g = torch.Generator().manual_seed(3)
    for cols in (1000, 777, 1024):
        x = torch.randn(33, cols, generator=g).to(cuda)
        torch.testing.assert_close(fn(x), torch.softmax(x, -1), rtol=1e-5, atol=1e-6)
    with pytest.raises(RuntimeError):
        fn(torch.randn(33, 5000, generator=g).to(cuda))
    torch.cuda.synchronize()


@pytest.mark.parametrize("shape,dtype,split", [((1, 65536, 128), torch.float32, True),
                                               ((4, 8192, 256), torch.bfloat16, True),
                                               ((2, 4096, 72), torch.float32, None),
                                               ((512, 256, 64), torch.float16, False)])
def test_outer_reduction_split_over_a_cluster(cuda, shape, dtype, split):
    """A long reduced axis over a small kept extent: the generated outer mapping gives each
    tile to a cluster of CTAs whose partial vectors meet in rank 0's shared memory
    (distributed shared memory, no scratch in global memory).  Parity with fp64 eager."""
    g = torch.Generator().manual_seed(shape[1])
    x = torch.randn(*shape, generator=g).to(dtype).to(cuda)
    for op in (torch.sum, torch.amax):
        out, code = compile_and_code(lambda t: op(t, 1), x)
        if split is not None:
            assert ("launch_outer_split_gen<" in code) == split
        exp = op(x.double(), 1)
        if op is torch.amax:
            assert torch.equal(out.double(), exp)
        else:
            tol = 2e-5 if dtype == torch.float32 else 2e-2
            assert graphs.max_rel_err(out.cpu(), exp.cpu(), floor=float(exp.abs().mean())) <= tol


def test_accumulating_scatters_use_atomic_adds(cuda):
    """index_put(accumulate=True), index_add and scatter_add are generated (store mode
    atomic_add) rather than left to extern kernels; integer accumulation is exact, float
    accumulation agrees with eager up to the order of the additions."""
    g = torch.Generator().manual_seed(29)
    idx = torch.randint(0, 100, (5000,), generator=g).to(cuda)
    vals = torch.randn(5000, 16, generator=g).to(cuda)
    base = torch.randn(100, 16, generator=g).to(cuda)
    out, code = compile_and_code(lambda t, i, v: t.index_put((i,), v, accumulate=True), base, idx, vals)
    assert "scatter_add(" in code
    torch.testing.assert_close(out, base.index_put((idx,), vals, accumulate=True), rtol=1e-4, atol=1e-4)
    out, code = compile_and_code(lambda t, i, v: torch.index_add(t, 0, i, v), base, idx, vals)
    torch.testing.assert_close(out, torch.index_add(base, 0, idx, vals), rtol=1e-4, atol=1e-4)
    idx2 = torch.randint(0, 100, (5000, 16), generator=g).to(cuda)
    out, code = compile_and_code(lambda t, i, v: torch.scatter_add(t, 0, i, v), base, idx2, vals)
    torch.testing.assert_close(out, torch.scatter_add(base, 0, idx2, vals), rtol=1e-4, atol=1e-4)
    counts = torch.zeros(100, dtype=torch.int64, device=cuda)
    ones = torch.ones(5000, dtype=torch.int64, device=cuda)
    out, _ = compile_and_code(lambda t, i, v: t.index_put((i,), v, accumulate=True), counts, idx, ones)
    assert torch.equal(out, torch.bincount(idx, minlength=100))


def test_bandwidth_debug_print(cuda, capsys):
    """config.profile_bandwidth: one 'ms  GB  GB/s' line per generated launch, the bytes being
    those of the tensor arguments (the reference's debug autotuner prints the same three
    figures, inductor_x/npu_triton_heuristics.py:274-299)."""
    import re

    from inductor_x_b200 import config

    x = torch.randn(2048, 4096, device=cuda)
    fn = torch.compile(lambda t: torch.relu(t) * 2.0)
    torch._dynamo.reset()
    fn(x)
    capsys.readouterr()
    config.profile_bandwidth = True
    try:
        fn(x)
        torch.cuda.synchronize()
    finally:
        config.profile_bandwidth = False
    out = capsys.readouterr().out
    m = re.search(r"([\d.]+)ms\s+([\d.]+)GB\s+([\d.]+)GB/s", out)
    assert m, out
    assert abs(float(m.group(2)) - 2 * x.numel() * 4 / 1e9) < 1e-3      # one read and one write of x
    assert float(m.group(3)) > 100.0


def test_float64_graphs_are_refused_not_narrowed(cuda):
    from inductor_x_b200.codegen.kernel import UnsupportedByTemplates

    x = torch.randn(64, 128, dtype=torch.float64, device=cuda)
    torch._dynamo.reset()
    with pytest.raises(Exception) as e:
        torch.compile(lambda t: (t * 2 + 1).sum(-1))(x)
    assert "float64" in str(e.value) or isinstance(e.value, UnsupportedByTemplates)


def test_debug_build_reports_an_out_of_range_index(cuda):
    """With config.debug_bounds every data-dependent index is checked on the device: the
    violation is counted, the access is redirected to element 0 (nothing faults) and the
    launcher raises IndexError on the host."""
    from inductor_x_b200 import config

    table = torch.arange(100 * 8, dtype=torch.float32, device=cuda).view(100, 8)
    good = torch.tensor([0, 5, 99, 17], device=cuda)
    bad = torch.tensor([0, 5, 100, 17], device=cuda)
    fn = lambda t, i: torch.ops.aten.index.Tensor(t, [i]) * 2.0
    config.debug_bounds = True
    try:
        out, code = compile_and_code(fn, table, good)
        assert "checked_index(" in code and "bounds=True" in code
        assert torch.equal(out, table[good] * 2.0)
        with pytest.raises(IndexError):
            torch.compile(fn)(table, bad)
        torch.cuda.synchronize()          # the context is still usable
        assert torch.equal(torch.compile(fn)(table, good), table[good] * 2.0)
    finally:
        config.debug_bounds = False
        torch._dynamo.reset()


def test_llama_decoder_layer_compiles_to_templates(cuda):
    """Configuration 5 at reduced width: hidden 512, 4 heads of 128, FFN 1376, 2 x 256 tokens."""
    from inductor_x_b200.llama_layer import decoder_layer

    w = inputs.c5_weights(hidden=512, heads=4, ffn=1376, seed=0)
    x = inputs.c5_input(2, 256, 512, seed=1)
    cos, sin = inputs.rope_tables(256, 128)
    wd = {k: v.to(cuda) for k, v in w.items()}
    fn = lambda x, cos, sin: decoder_layer(x, wd, cos, sin, heads=4)
    out, code = compile_and_code(fn, x.to(cuda), cos.to(cuda), sin.to(cuda))
    assert "b200_sdpa" in code and "ixb_load_kernel" in code
    assert "triton_" not in code.replace("triton_helpers", "")
    exp = graphs.llama_layer(x, w, heads=4, compute=torch.float64)
    assert graphs.max_rel_err(out.cpu(), exp) <= 2e-2
    eager = fn(x.to(cuda), cos.to(cuda), sin.to(cuda))
    assert graphs.max_rel_err(out.cpu(), eager.cpu()) <= 2e-2


# ---- graphs modelled on the reference's own compile-vs-eager tests (test/npu_indexing) ----
@pytest.mark.parametrize("dim", [0, 1, 2, 3])
@pytest.mark.parametrize("perm", [(0, 1, 3, 2), (0, 2, 1, 3), (2, 1, 0, 3), (3, 1, 2, 0), (1, 0, 2, 3)])
def test_reduction_broadcast_permute(cuda, dim, perm):
    """sum over one dim, broadcast back, permute (reduction_broadcast_permute_test.py:20-33)."""
    x = torch.randn(8, 8, 64, 32, generator=torch.Generator().manual_seed(dim)).to(cuda)
    fn = lambda t: (t - t.sum(dim, keepdim=True)).permute(*perm).contiguous()
    out, _ = compile_and_code(fn, x)
    torch.testing.assert_close(out, fn(x), rtol=1e-4, atol=1e-4)


def test_rearrange_b_n_s_d_to_s_b_nd(cuda):
    """'b n s d -> s b (n d)' (permute_reshape_test.py:9-31)."""
    x = torch.randn(4, 8, 96, 64, generator=torch.Generator().manual_seed(2)).to(cuda)
    fn = lambda t: (t * 2.0).permute(2, 0, 1, 3).reshape(96, 4, 512)
    out, _ = compile_and_code(fn, x)
    assert torch.equal(out, fn(x))


@pytest.mark.parametrize("dims", [(0,), (1,), (2,), (0, 2), (1, 2), (0, 1, 2)])
def test_var_mean_axis_sets(cuda, dims):
    """var_mean over several axis sets (var_mean_test.py:28-36)."""
    x = torch.randn(16, 24, 40, generator=torch.Generator().manual_seed(len(dims))).to(cuda)
    (var, mean), _ = compile_and_code(lambda t: torch.var_mean(t, dims), x)
    ev, em = torch.var_mean(x.double(), dims)
    torch.testing.assert_close(var.double(), ev, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(mean.double(), em, rtol=1e-4, atol=1e-5)


def test_repeat_and_unaligned_argmax(cuda):
    """repeat (repeat_test.py:28-31) and argmax on unaligned shapes (argmax_unalign_test.py:36-55)."""
    x = torch.randn(3, 513, generator=torch.Generator().manual_seed(9)).to(cuda)
    out, _ = compile_and_code(lambda t: t.repeat(2, 3) + 1, x)
    assert torch.equal(out, x.repeat(2, 3) + 1)
    for shape in [(513, 64), (7, 1023), (129, 300)]:
        y = torch.randn(*shape, generator=torch.Generator().manual_seed(shape[0])).to(cuda)
        idx, _ = compile_and_code(lambda t: torch.argmax(t, -1), y)
        assert torch.equal(idx, torch.argmax(y, -1))


def test_mamba_split_permute(cuda):
    """split + permute + elementwise of the mamba regression graph (mamba_test.py:7-29)."""
    x = torch.randn(4, 64, 96, generator=torch.Generator().manual_seed(11)).to(cuda)

    def fn(t):
        a, b, c = torch.split(t, [32, 32, 32], dim=-1)
        return (F.silu(a) * b + c).permute(0, 2, 1).contiguous()

    out, _ = compile_and_code(fn, x)
    torch.testing.assert_close(out, fn(x), rtol=1e-5, atol=1e-5)


def test_context_parallel_softmax_merge(cuda):
    """Online-softmax merge of two attention partials, the per-step math of ring attention
    (attn_cp_test.py:36-59 forward_update)."""
    g = torch.Generator().manual_seed(13)
    prev_out, cur_out = (torch.randn(2, 4, 128, 64, generator=g).to(cuda) for _ in range(2))
    prev_max, cur_max = (torch.randn(2, 4, 128, 1, generator=g).to(cuda) for _ in range(2))
    prev_sum, cur_sum = (torch.rand(2, 4, 128, 1, generator=g).to(cuda) + 0.5 for _ in range(2))

    def forward_update(po, pm, ps, co, cm, cs):
        m = torch.maximum(pm, cm)
        ps2 = ps * torch.exp(pm - m)
        cs2 = cs * torch.exp(cm - m)
        s = ps2 + cs2
        return po * (ps2 / s) + co * (cs2 / s), m, s

    outs, _ = compile_and_code(forward_update, prev_out, prev_max, prev_sum, cur_out, cur_max, cur_sum)
    for a, e in zip(outs, forward_update(prev_out, prev_max, prev_sum, cur_out, cur_max, cur_sum)):
        torch.testing.assert_close(a, e, rtol=1e-5, atol=1e-5)


def test_accuracy_check_walks_every_intermediate_of_config_2():
    """The per-intermediate harness on the softmax -> LayerNorm chain: every node Dynamo
    captured is produced by the generated kernels (all intermediates are graph outputs) and
    agrees with eager within the 16-bit tolerance."""
    from inductor_x_b200 import accuracy_check as ac

    d = inputs.c2(64, 4096, seed=3)
    x, g, ga, be = (d[k].cuda() for k in ("x", "g", "gamma", "beta"))
    rep = ac.check(lambda x, g, ga, be: F.layer_norm(torch.softmax(x, -1) * g + x, (4096,), ga, be, 1e-5),
                   x, g, ga, be)
    assert len(rep.records) >= 4, rep.format()
    assert rep.ok, rep.format()
    assert all(r.compiled_md5 is not None for r in rep.records)


def _top2_gating(logits, capacity: int):
    """Top-2 expert gating in the style of the reference's MoE workload
    (test/npu_indexing/moe/run_moe.py:24-112): softmax over experts, top-2 choice, one-hot
    masks, running positions inside each expert's capacity buffer (cumsum), capacity cut,
    renormalised gate weights and flattened (expert, slot) indices."""
    probs = torch.softmax(logits, dim=1)
    n_exp = probs.shape[1]
    _, chosen = torch.topk(probs, 2, dim=-1)
    mask = F.one_hot(chosen, num_classes=n_exp)
    first, second = mask[:, 0, :], mask[:, 1, :]
    pos1 = torch.cumsum(first, dim=0) - 1
    pos2 = torch.cumsum(second, dim=0) - 1 + torch.sum(first, dim=0, keepdim=True)
    aux = torch.mean(probs, dim=0) * torch.mean(first.float(), dim=0)
    l_aux = aux.sum() * n_exp
    first = first * torch.lt(pos1, capacity)
    second = second * torch.lt(pos2, capacity)
    slot1 = torch.sum(pos1 * first, dim=1)
    slot2 = torch.sum(pos2 * second, dim=1)
    w1, e1 = torch.max(probs * first.float(), dim=1)
    w2, e2 = torch.max(probs * second.float(), dim=1)
    denom = torch.clamp(w1 + w2, min=torch.finfo(probs.dtype).eps)
    flat = torch.cat([e1.int() * capacity + slot1.int(), e2.int() * capacity + slot2.int()], dim=0)
    weights = torch.cat([w1 / denom, w2 / denom], dim=0)
    return l_aux, flat, weights


@pytest.mark.parametrize("tokens,experts", [(4096, 16), (1000, 8)])
def test_moe_top2_gating_graph(tokens, experts):
    """Scan / top-k stay extern kernels, everything between them (softmax, one-hot masks,
    integer sums along both axes, max with index, clamp, integer index arithmetic, cat) is
    generated.  Integer outputs must be exact, float outputs within the fp32 tolerance."""
    g = torch.Generator().manual_seed(tokens + experts)
    logits = torch.randn(tokens, experts, generator=g).cuda()
    capacity = max(4, 2 * tokens // experts)
    want = _top2_gating(logits, capacity)
    torch._dynamo.reset()
    got = torch.compile(_top2_gating)(logits, capacity)
    assert graphs.max_rel_err(got[0].cpu(), want[0].cpu()) <= 1e-5
    assert torch.equal(got[1].cpu(), want[1].cpu())
    assert graphs.max_rel_err(got[2].cpu(), want[2].cpu()) <= 1e-5


def test_vocabulary_sized_row():
    """log_softmax over a 128,256-wide fp32 row (a Llama-3 vocabulary): longer than a team
    holds in registers, so the row is walked in chunks (one loop for the online maximum and
    sum, one for the output) - still one kernel."""
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(24, 128256, generator=g) * 3).cuda()
    torch._dynamo.reset()
    got, code = compile_and_code(lambda t: torch.log_softmax(t, -1), x)
    assert code.count("ixb_load_kernel('''") == 1 and code.count("c.nchunks()") == 2
    want = torch.log_softmax(x.double(), -1)
    assert graphs.max_rel_err(got.cpu().double(), want.cpu()) <= 1e-5


def test_rows_longer_than_a_team_are_walked_in_chunks(cuda):
    """Looped inner reductions (inductor_x/codegen/triton.py:1208-1253): any row length
    compiles; sums, extrema, arg-reductions, variance and a LayerNorm chain over rows of
    100,000 to 1,048,576 elements against fp64 eager, integers exactly."""
    g = torch.Generator().manual_seed(41)
    x = torch.randn(4, 300000, generator=g).to(cuda)
    (var, mean), code = compile_and_code(lambda t: torch.var_mean(t, -1), x)
    assert "c.nchunks()" in code
    ev, em = torch.var_mean(x.double(), -1)
    assert graphs.max_rel_err(var.cpu(), ev.cpu()) <= 1e-5
    assert graphs.max_rel_err(mean.cpu(), em.cpu(), floor=0.01) <= 1e-4
    idx, _ = compile_and_code(lambda t: (torch.argmax(t, -1), torch.amin(t, -1)), x)
    assert torch.equal(idx[0], torch.argmax(x, -1)) and torch.equal(idx[1], torch.amin(x, -1))
    ones = torch.ones(3, 1 << 20, dtype=torch.int32, device=cuda) * 4096      # row sums of 2^32
    s, _ = compile_and_code(lambda t: t.sum(-1, dtype=torch.int64), ones)
    assert s.tolist() == [1 << 32] * 3
    xb = (torch.randn(16, 100000, generator=g) * 2).bfloat16().to(cuda)
    ga, be = (torch.randn(100000, generator=g).bfloat16().to(cuda) for _ in range(2))
    out, code = compile_and_code(lambda t, a, b: F.layer_norm(t, (100000,), a, b), xb, ga, be)
    assert code.count("ixb_load_kernel('''") == 1
    want = F.layer_norm(xb.double(), (100000,), ga.double(), be.double())
    assert graphs.max_rel_err(out.cpu().double(), want.cpu()) <= 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(64, 1024), (37, 1000), (8, 4096), (300, 24), (5, 16384), (3, 7, 130)])
def test_cumsum_over_the_last_axis_is_scanned_on_chip(cuda, dtype, shape):
    """cumsum along the stride-1 axis: one row kernel with a team-wide prefix sum, fused with
    the pointwise work before and after it (the reference leaves cumsum to an extern kernel,
    inductor_x/lowering.py:235-245).  fp32 accumulation: rel 1e-5 for fp32, 2e-2 for bf16,
    against a float64 scan of the same (rounded) inputs; ragged rows, sub-warp teams and rows
    of 16384 elements (1024 threads x 4 vectors) included."""
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(*shape, generator=g).to(dtype)
    fn = lambda t: torch.cumsum(t * 0.5, -1) + 1.0
    got, code = compile_and_code(fn, x.to(cuda))
    assert code.count("ixb_load_kernel('''") == 1 and "c.template scan<ixb::SumOp>(" in code
    assert "torch.ops.aten.cumsum.default(" not in code
    want = torch.cumsum(x.double() * 0.5, -1) + 1.0
    assert got.dtype == dtype
    assert graphs.max_rel_err(got.cpu().double(), want) <= graphs.tolerance(dtype)


@pytest.mark.parametrize("shape", [(1, 16384), (2, 16384), (4, 12000), (16384,)])
def test_long_cumsum_of_few_rows_fuses_with_the_reduction_after_it(cuda, shape):
    """Few kept rows and a long scanned axis: Inductor's heuristic would cut the scan in two;
    here it stays one row kernel, and the row sum that consumes it joins the same kernel."""
    g = torch.Generator().manual_seed(sum(shape) + 3)
    x = torch.randn(*shape, generator=g)
    got, code = compile_and_code(lambda t: (torch.cumsum(t, -1) * 0.25).sum(-1), x.to(cuda))
    assert code.count("ixb_load_kernel(" + "'" * 3) == 1 and "c.template scan<ixb::SumOp>(" in code
    want = (torch.cumsum(x.double(), -1) * 0.25).sum(-1)
    # the row sum of a running sum cancels heavily: absolute bound scaled by the row's magnitude
    scale = torch.cumsum(x.double(), -1).abs().sum(-1) * 0.25
    assert ((got.cpu().double() - want).abs() <= 1e-5 * scale).all()


def test_cumsum_along_other_axes_stays_extern(cuda):
    x = torch.randn(512, 64, device=cuda)
    got, code = compile_and_code(lambda t: torch.cumsum(t, 0) * 2.0, x)
    assert "torch.ops.aten.cumsum.default(" in code and "c.template scan" not in code
    torch.testing.assert_close(got, torch.cumsum(x, 0) * 2.0, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32, torch.bool])
@pytest.mark.parametrize("shape", [(33, 1000), (4, 8192), (129, 24)])
def test_integer_cumsum_over_the_last_axis_is_exact(cuda, dtype, shape):
    """Integer, index and boolean rows are scanned with 64-bit sums: bit-exact, including
    values far above 2^24 (where an fp32 accumulator would round)."""
    g = torch.Generator().manual_seed(sum(shape) + 1)
    if dtype == torch.bool:
        x = torch.rand(*shape, generator=g) > 0.5
    elif dtype == torch.int32:
        x = torch.randint(-(2 ** 30), 2 ** 30, shape, generator=g, dtype=torch.int32)
    else:
        x = torch.randint(-(2 ** 40), 2 ** 40, shape, generator=g, dtype=torch.int64)
    got, code = compile_and_code(lambda t: torch.cumsum(t, -1), x.to(cuda))
    assert "c.template scan_int<typename Ctx::ISum>(" in code and "torch.ops.aten.cumsum.default(" not in code
    want = torch.cumsum(x, -1)
    assert got.dtype == torch.int64 and torch.equal(got.cpu(), want)


@pytest.mark.parametrize("shape", [(64, 1024), (37, 1000), (300, 24)])
def test_cumprod_over_the_last_axis(cuda, shape):
    """The same team-wide scan with the product operator (values near 1 so that long rows
    neither overflow nor vanish); rel 1e-5 against a float64 scan."""
    g = torch.Generator().manual_seed(sum(shape) + 7)
    x = 1.0 + 0.01 * torch.randn(*shape, generator=g)
    got, code = compile_and_code(lambda t: torch.cumprod(t, -1), x.to(cuda))
    assert "c.template scan<ixb::ProdOp>(" in code and "torch.ops.aten.cumprod.default(" not in code
    assert graphs.max_rel_err(got.cpu().double(), torch.cumprod(x.double(), -1)) <= 1e-5


def test_integer_bit_operations_match_eager(cuda):
    """Bitwise ops, shifts, narrowing conversions and overflowing sums / products of integers:
    bit-exact against eager mode (integers are carried in 64 bits and wrapped back where the
    result can leave the range of its type)."""
    g = torch.Generator().manual_seed(11)
    a = torch.randint(-(2 ** 40), 2 ** 40, (5000,), generator=g)
    b = torch.randint(0, 40, (5000,), generator=g)
    fn = lambda a, b: ((a & (b * 977)) | (a ^ 0x5555)) + (~a) + (a << b) + (a >> b)
    got, code = compile_and_code(fn, a.to(cuda), b.to(cuda))
    assert "ixb::gen::op::bit_and(" in code and "logical_" not in code
    assert torch.equal(got.cpu(), fn(a, b))
    a32 = torch.randint(-(2 ** 31), 2 ** 31 - 1, (5000,), generator=g, dtype=torch.int32)
    b32 = torch.randint(0, 31, (5000,), generator=g, dtype=torch.int32)

    def narrow(a, b):
        return ((a << b) + a * 1103515245 - b, (~a.to(torch.uint8)).float(),
                a.to(torch.int8).to(torch.int64) + a.to(torch.int16), (a > 0) ^ (b > 15))

    got, code = compile_and_code(narrow, a32.to(cuda), b32.to(cuda))
    assert "wrap_int<32, true>(" in code and "wrap_int<8, false>(" in code
    for o, w in zip(got, narrow(a32, b32)):
        assert o.dtype == w.dtype and torch.equal(o.cpu(), w)


def test_padding_pooling_and_dropout(cuda):
    """A constant pad feeding a strided max-pool (masked sub-blocks) against eager mode, and a
    training-mode dropout: the random mask comes from ATen's generator, the scaling around it is
    generated, the same seed gives the same result."""
    g = torch.Generator().manual_seed(12)
    x = torch.randn(2, 3, 33, 31, generator=g)
    fn = lambda t: F.max_pool2d(F.pad(t, (1, 2, 3, 4), value=-1.0) * 2.0, 3, 2, 1)
    got, code = compile_and_code(fn, x.to(cuda))
    assert "= torch.ops.aten.constant_pad_nd.default(" not in code
    torch.testing.assert_close(got.cpu(), fn(x), rtol=1e-6, atol=1e-6)
    y = torch.rand(256, 1024, generator=g) + 0.5
    drop = torch.compile(lambda t: F.dropout(t * 2.0, 0.25, True) + 1.0)
    torch.manual_seed(5)
    o1 = drop(y.to(cuda))
    torch.manual_seed(5)
    o2 = drop(y.to(cuda))
    assert torch.equal(o1, o2)
    kept = o1.cpu() != 1.0
    assert abs(kept.float().mean().item() - 0.75) < 0.01
    torch.testing.assert_close(o1.cpu()[kept], (y * 2.0 / 0.75 + 1.0)[kept], rtol=1e-5, atol=1e-5)


def test_inverse_hyperbolic_and_extern_special_functions(cuda):
    """asinh / acosh / atanh / erfinv / nextafter / ldexp are generated (rel 1e-5 against float64);
    digamma, i0 and logcumsumexp stay extern kernels inside a compiled graph."""
    g = torch.Generator().manual_seed(13)
    x = torch.rand(64, 300, generator=g) * 0.8 + 0.1
    fn = lambda t: (torch.asinh(t) + torch.acosh(t + 1) + torch.atanh(t) + torch.erfinv(t)
                    + torch.nextafter(t, t + 1) + torch.ldexp(t, torch.tensor(3, device=t.device)))
    got, code = compile_and_code(fn, x.to(cuda))
    assert code.count("ixb_load_kernel('''") == 1 and "ixb::gen::op::erfinv(" in code
    want = (torch.asinh(x.double()) + torch.acosh(x.double() + 1) + torch.atanh(x.double()) + torch.erfinv(x.double())
            + x.double() + x.double() * 8)
    assert graphs.max_rel_err(got.cpu().double(), want) <= 1e-5
    fn = lambda t: torch.logcumsumexp(torch.digamma(t) * 2.0, -1) + torch.special.i0(t)
    got, code = compile_and_code(fn, x.to(cuda))
    assert "torch.ops.aten.digamma.default(" in code and "torch.ops.aten.logcumsumexp.default(" in code
    torch.testing.assert_close(got.cpu(), fn(x), rtol=1e-4, atol=1e-5)


def _zoo_inputs():
    g = torch.Generator().manual_seed(14)
    x = torch.randn(4099, generator=g) * 3
    y = torch.randn(4099, generator=g) * 2
    y[y.abs() < 0.05] = 0.7
    x[:8] = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 1e10, -1e10])        # round-half-even, huge ratios
    i = torch.randint(-50, 50, (4099,), generator=g)
    j = torch.randint(-7, 8, (4099,), generator=g)
    j[j == 0] = 3
    return x, y, i, j


def test_floating_pointwise_ops_match_eager(cuda):
    """One kernel per family of floating pointwise ops (several outputs each) against eager mode on
    the same inputs: rounding modes, signs of remainder / fmod / floor division, NaN handling of
    maximum / minimum / clamp / relu, selects, the transcendental set."""
    x, y, _, _ = _zoo_inputs()
    xn = x.clone()
    xn[100:110] = float("nan")

    def rounding(a, b):
        return (torch.round(a), torch.trunc(a), torch.floor(a), torch.ceil(a), torch.sign(a), torch.remainder(a, b),
                torch.fmod(a, b), torch.floor_divide(a, b), torch.div(a, b, rounding_mode="trunc"), torch.copysign(a, b))

    def nans(a, b):
        return (torch.maximum(a, b), torch.minimum(a, b), a.clamp(-1.0, 1.0), torch.relu(a), torch.where(a > b, a, b),
                torch.isnan(a), torch.nan_to_num(a, nan=2.0), (a != a) | (b > 0), torch.hypot(a, b), torch.atan2(a, b))

    def transcendental(a):
        p = a.abs() + 0.1
        return (torch.exp(a * 0.3), torch.expm1(a * 0.1), torch.log(p), torch.log2(p), torch.log10(p), torch.log1p(p),
                torch.sqrt(p), torch.rsqrt(p), torch.sin(a), torch.cos(a), torch.tan(a.clamp(-1.2, 1.2)), torch.tanh(a),
                torch.sigmoid(a), torch.erf(a), torch.erfc(a), torch.sinh(a * 0.5), torch.cosh(a * 0.5),
                torch.atan(a), torch.asin(a.clamp(-1, 1) * 0.99), torch.acos(a.clamp(-1, 1) * 0.99), torch.exp2(a * 0.5),
                torch.pow(p, 1.7), torch.pow(p, b_const), torch.lgamma(p), torch.reciprocal(p), torch.square(a),
                F.gelu(a), F.silu(a), F.softplus(a), torch.abs(a), -a)

    b_const = 3
    for fn, args, tol in ((rounding, (x, y), 1e-6), (nans, (xn, y), 1e-6), (transcendental, (x[8:],), 2e-5)):
        got, code = compile_and_code(fn, *(a.to(cuda) for a in args))
        want = fn(*(a.double() if tol > 1e-6 else a for a in args))
        for k, (o, w) in enumerate(zip(got, want)):
            assert o.shape == w.shape, (fn.__name__, k)
            if w.dtype == torch.bool:
                assert torch.equal(o.cpu(), w), (fn.__name__, k)
            else:
                torch.testing.assert_close(o.cpu().double(), w.double(), rtol=tol, atol=tol, equal_nan=True,
                                           msg=lambda m, k=k: f"{fn.__name__} output {k}: {m}")


def test_integer_pointwise_ops_match_eager(cuda):
    """Integer arithmetic with negative operands (floor division, remainder, truncating division,
    fmod, abs, sign, min / max, clamp, selects, comparisons, powers, conversions): bit-exact."""
    x, _, i, j = _zoo_inputs()

    def ints(a, b):
        return (a // b, a % b, torch.div(a, b, rounding_mode="trunc"), torch.fmod(a, b), a.abs(), torch.sign(a),
                torch.maximum(a, b), torch.minimum(a, b), a.clamp(-10, 10), torch.where(a > b, a, b), a * b - a,
                (a >= b) & (a != 3), a ** 2, -a, a / b, (a.float() * 0.37).to(torch.int64), a.to(torch.int16) * 1000,
                (a + 200).to(torch.uint8) + 100, a.to(torch.bool), (a > 0).to(torch.int32) + a.to(torch.int32))

    got, code = compile_and_code(ints, i.to(cuda), j.to(cuda))
    for k, (o, w) in enumerate(zip(got, ints(i, j))):
        assert o.dtype == w.dtype, k
        if w.dtype.is_floating_point:
            torch.testing.assert_close(o.cpu(), w, rtol=1e-6, atol=1e-6)
        else:
            assert torch.equal(o.cpu(), w), k
    # float -> int truncates toward zero
    got, _ = compile_and_code(lambda t: ((t * 3).to(torch.int32), (t * 3).to(torch.int64) // 2), x[8:].to(cuda))
    want = ((x[8:] * 3).to(torch.int32), (x[8:] * 3).to(torch.int64) // 2)
    for o, w in zip(got, want):
        assert torch.equal(o.cpu(), w)


def test_integer_argmax_compares_integers(cuda):
    """argmax / argmin of 64-bit integers whose differences vanish in fp32 (values near 2^40,
    all distinct): the indices equal eager mode's, over the last axis, over the first axis and
    over a row long enough to be walked in chunks."""
    g = torch.Generator().manual_seed(15)
    x = torch.randperm(37 * 1000, generator=g).reshape(37, 1000) + (1 << 40)
    fn = lambda t: (t.argmax(-1), t.argmin(-1), t.argmax(0))
    got, code = compile_and_code(fn, x.to(cuda))
    assert "reduce_arg_int<true>(" in code and "reduce_arg_int<false>(" in code
    for o, w in zip(got, fn(x)):
        assert torch.equal(o.cpu(), w)
    y = torch.randperm(3 * 70001, generator=g).reshape(3, 70001) + (1 << 40)
    got, code = compile_and_code(lambda t: t.argmin(-1), y.to(cuda))
    assert "xreduce_arg_int<false>(" in code
    assert torch.equal(got.cpu(), y.argmin(-1))
