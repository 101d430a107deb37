"""The graphs of the reference's own regression scripts (test/npu_indexing/issue*_test.py,
clamp_test.py, reduction_test.py, pointwise_test.py, written/test_slice.py,
test_AddLayerNorm.py), restated with the same operators, dtypes and - where they are cheap -
the same shapes.  Each script compiles a function with the Inductor backend and compares with
eager mode at rtol = atol = 1e-3; the GPU tests here do the same through this backend (with the
tolerance tightened to what fp32 / fp16 arithmetic gives), and the CPU test checks that every
graph is instantiated from the templates without a Triton kernel.  Collected last so that a
failure here cannot mask other tests."""
import pytest
import torch
import torch.nn.functional as F


def issue70(x):
    """mean over the last axis of a single row of 7168 (issue70_test.py:8-19)."""
    return x.mean(-1)


def issue62(addmm, add):
    """Six-way split of a projection, LayerNorm without affine over 1536 fp16 columns computed in
    fp32, scaled by (1 + chunk 1) and shifted by chunk 0, both broadcast over the sequence
    (issue62_test.py:8-33)."""
    chunks = torch.split(addmm, 1536, 1)
    x = add.contiguous().float()
    var, mean = torch.var_mean(x, [2], correction=0, keepdim=True)
    normed = ((add - mean) * torch.rsqrt(var + 1e-6)).half()
    return normed * (chunks[1].unsqueeze(1) + 1) + chunks[0].unsqueeze(1)


def issue57(view, embedding, bias):
    """A [512, 512, 64] table permuted to [64, 512, 512], plus a row bias, plus a contiguous
    operand (issue57_test.py:10-17)."""
    return view + (embedding.permute(2, 0, 1).unsqueeze(0) + bias)


def issue59(x, y, z):
    """LayerNorm of a single row written with full reductions and numel() divisors
    (issue59_test.py:8-20)."""
    total = torch.sum(x)
    mean = total / torch.numel(total)
    sub = x - mean
    total_sq = torch.sum(sub * sub)
    rstd = torch.rsqrt(total_sq / torch.numel(total_sq) + 1e-5)
    mul = sub * rstd
    return mul, mul * y + z, rstd / torch.numel(rstd)


def issue61(view, embedding):
    """The permuted table sliced from -128 along the query axis, added, viewed twice
    (issue61_test.py:19-30)."""
    sliced = embedding.permute(2, 0, 1).unsqueeze(0)[:, :, -128:, :]
    return (view + sliced).view(-1, 128, 128).view(-1, 6, 128, 128)


def issue54(x, wq, bq, bk, wk_t, wv, bv):
    """Three projections of one activation, head split by view + permute, contiguous copies in
    the layouts a batched matmul wants, Q K^T (issue54_test.py:8-36; batch 8 instead of 64)."""
    b = x.shape[0] // 512
    q = torch.addmm(bq, x, wq.t()).view(b, 512, 4, 64).permute(0, 2, 1, 3)
    k = torch.addmm(bk, x, wk_t).view(b, 512, 4, 64).permute(0, 2, 1, 3)
    v = torch.addmm(bv, x, wv.t()).view(b, 512, 4, 64).permute(0, 2, 1, 3)
    qc = q.expand(b, 4, 512, 64).clone(memory_format=torch.contiguous_format).view(b * 4, 512, 64)
    kc = k.permute(0, 1, 3, 2).expand(b, 4, 64, 512).clone(memory_format=torch.contiguous_format).view(b * 4, 64, 512)
    vc = v.expand(b, 4, 512, 64).clone(memory_format=torch.contiguous_format).view(b * 4, 512, 64)
    return torch.bmm(qc, kc), vc


def add_layernorm(a, b):
    """x = a + b normalised over the last axis with the deviation (not the variance) plus eps in
    the denominator, as the hand-written kernel of test_AddLayerNorm.py:19-60 computes it."""
    x = a + b
    mean = x.mean(-1, keepdim=True)
    sub = x - mean
    return sub / (torch.sqrt((sub * sub).mean(-1, keepdim=True)) + 1e-5)


def clamp_tensor_bounds(x, lo, hi):
    """clamp with tensor bounds (clamp_test.py:20-31)."""
    return x.clamp(lo, hi)


def slice_clone_assign_update(x, col, out):
    """Column 0 cloned out of a [16, 32] tensor, a vector assigned to column 2 and added to
    column 3 of another (written/test_slice.py:10-60)."""
    out = out.clone()
    out[..., 2] = col
    out[..., 3] += col
    return x[..., 0].clone(), out


def add_then_reduce(a, b, dim):
    """(a + b).sum(dim) (reduction_test.py:6-13)."""
    return (a + b).sum(dim)


CASES = {
    # name: (function, argument maker, tolerance relative to max(|expected|, 1); 0 = bit-exact)
    "issue70": (issue70, lambda rn, ri: (rn(1, 1, 7168),), 1e-5),
    "issue62": (issue62, lambda rn, ri: (rn(2, 9216, dtype=torch.float16), rn(2, 1024, 1536, dtype=torch.float16)), 4e-3),
    "issue57": (issue57, lambda rn, ri: (rn(1, 64, 512, 512), rn(512, 512, 64), rn(1, 1, 1, 512)), 1e-5),
    "issue59": (issue59, lambda rn, ri: (rn(1, 1024), rn(1, 1024), rn(1, 1024)), 1e-4),
    "issue61": (issue61, lambda rn, ri: (rn(64, 6, 128, 128), rn(128, 128, 6)), 1e-5),
    "issue54": (issue54, lambda rn, ri: (rn(8 * 512, 256), rn(256, 256) * 0.05, rn(256), rn(256), rn(256, 256) * 0.05,
                                         rn(256, 256) * 0.05, rn(256)), 1e-3),
    "add_layernorm": (add_layernorm, lambda rn, ri: (rn(64, 512, 256), rn(64, 512, 256)), 1e-4),
    "clamp_f32": (clamp_tensor_bounds, lambda rn, ri: (rn(1024, 32), rn(1024, 32) - 1, rn(1024, 32) + 1), 0.0),
    "clamp_bf16": (clamp_tensor_bounds, lambda rn, ri: (rn(1024, 32, dtype=torch.bfloat16),
                                                        rn(1024, 32, dtype=torch.bfloat16) - 1,
                                                        rn(1024, 32, dtype=torch.bfloat16) + 1), 0.0),
    "clamp_i32": (clamp_tensor_bounds, lambda rn, ri: (ri(1024, 32, dtype=torch.int32), ri(1024, 32, dtype=torch.int32) - 50,
                                                       ri(1024, 32, dtype=torch.int32) + 50), 0.0),
    "clamp_i64": (clamp_tensor_bounds, lambda rn, ri: (ri(13), ri(13) - 50, ri(13) + 50), 0.0),
    "slices": (slice_clone_assign_update, lambda rn, ri: (rn(16, 32), rn(16, dtype=torch.float16),
                                                          rn(16, 32, dtype=torch.float16)), 0.0),
    "reduce_dim0": (lambda a, b: add_then_reduce(a, b, 0), lambda rn, ri: (rn(8, 16, 512, 64), rn(8, 16, 512, 64)), 1e-4),
    "reduce_dim2": (lambda a, b: add_then_reduce(a, b, 2), lambda rn, ri: (rn(8, 16, 512, 64), rn(8, 16, 512, 64)), 1e-4),
    "reduce_ragged": (lambda a, b: add_then_reduce(a, b, -1),
                      lambda rn, ri: (rn(2053, 1023, 7, 9), rn(2053, 1023, 7, 9)), 1e-4),
}


def _case(name, device):
    fn, make, tol = CASES[name]
    g = torch.Generator().manual_seed(57)

    def rn(*shape, dtype=torch.float32):
        return torch.randn(*shape, generator=g).to(dtype).to(device)

    def ri(*shape, dtype=torch.int64):
        return torch.randint(-100, 100, shape, generator=g).to(dtype).to(device)

    return fn, make(rn, ri), tol


def _compile(fn, args):
    from torch._inductor.utils import run_and_get_code

    torch._dynamo.reset()
    out, code = run_and_get_code(torch.compile(fn, dynamic=False), *args)
    text = "\n".join(code)
    assert "triton_" not in text.replace("triton_helpers", "").replace("triton_heuristics", "")
    return out, text


def test_regression_graphs_are_instantiated_from_the_templates(dry_backend):
    """Every graph compiles into template instantiations (built with nvcc, not launched); the
    ragged full-size case is left to the GPU run."""
    kernels = {}
    for name in CASES:
        if name == "reduce_ragged":
            continue
        fn, args, _ = _case(name, "cpu")
        _, code = _compile(fn, args)
        kernels[name] = code.count("ixb_load_kernel('''")
        assert kernels[name] >= 1, name
    # one kernel where the reference's Triton path also fuses everything
    assert kernels["issue70"] == 1 and kernels["issue57"] == 1 and kernels["issue61"] == 1
    assert kernels["issue62"] == 1 and kernels["add_layernorm"] == 1 and kernels["clamp_i64"] == 1


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
def test_regression_graphs_match_eager(cuda, name):
    fn, args, tol = _case(name, cuda)
    got, _ = _compile(fn, args)
    want = fn(*args)
    got = got if isinstance(got, (tuple, list)) else (got,)
    want = want if isinstance(want, (tuple, list)) else (want,)
    for o, w in zip(got, want):
        assert o.shape == w.shape and o.dtype == w.dtype, name
        if tol == 0.0:
            assert torch.equal(o, w), name
        else:
            scale = max(w.float().abs().max().item(), 1.0)
            assert (o.float() - w.float()).abs().max().item() <= tol * scale, name


@pytest.mark.gpu
def test_full_reduction_with_run_time_sizes(cuda):
    """A loss-style mean over every element of a tensor whose sizes are symbolic: one chunked row
    kernel serves both sizes (the launcher passes the reduced extent)."""
    g = torch.Generator().manual_seed(58)
    fn = torch.compile(lambda t: (t * t).mean(), dynamic=True)
    for shape in ((1000, 1024), (1500, 900), (64, 100)):
        x = torch.randn(*shape, generator=g).to(cuda)
        want = (x.double() * x.double()).mean()
        assert abs(fn(x).double().item() - want.item()) <= 1e-5 * abs(want.item())
