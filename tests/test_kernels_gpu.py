"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracle
and the committed golden vectors.

Bars: bit-exact for index / gather / max outputs; rel <= 1e-5 for fp32 reductions;
<= 2e-2 for bf16 / fp16 (relative to max(|expected|, rms(expected)))."""
import hashlib

import pytest
import torch

from inductor_x_b200 import ops
from inductor_x_b200 import runtime as rt
from oracle import c_oracle, graphs, inputs

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5
TOL_HALF = 2e-2


def dev(d, cuda):
    return {k: (v.to(cuda) if torch.is_tensor(v) else v) for k, v in d.items()}


# ------------------------------------------------------------------------ config 1
def test_c1_full_vs_golden(cuda, golden):
    d = dev(inputs.c1(), cuda)
    out = ops.affine_gelu_rowsum(d["x"], d["w"], d["b"]).cpu()
    assert graphs.max_rel_err(out, golden["c1_out_f64"]) <= TOL_F32
    assert graphs.max_rel_err(out, golden["c1_out_eager"]) <= TOL_F32


@pytest.mark.parametrize("rows,cols", [(1, 4), (3, 1023), (7, 1024), (513, 64), (64, 2048),
                                       (33, 4100), (5, 8192), (2, 16384), (130, 12)])
def test_c1_shapes_vs_oracle(cuda, rows, cols):
    d = inputs.c1(rows, cols, seed=rows * 31 + cols)
    exp = c_oracle.affine_gelu_rowsum(**d)
    out = ops.affine_gelu_rowsum(**dev(d, cuda)).cpu()
    assert graphs.max_rel_err(out, exp) <= TOL_F32


@pytest.mark.parametrize("team,vpt", [(32, 8), (64, 4), (128, 2), (256, 1), (256, 2), (1024, 4)])
def test_c1_every_config(cuda, team, vpt):
    d = inputs.c1(300, 1024, seed=5)
    exp = c_oracle.affine_gelu_rowsum(**d)
    dd = dev(d, cuda)
    try:
        out = ops.affine_gelu_rowsum(dd["x"], dd["w"], dd["b"], cfg={"team": team, "vpt": vpt}).cpu()
    except rt.IxbError as e:
        assert e.status == rt.IXB_ERR_UNSUPPORTED  # pair not instantiated
        return
    assert graphs.max_rel_err(out, exp) <= TOL_F32


def test_c1_empty(cuda):
    out = ops.affine_gelu_rowsum(torch.empty(0, 16, device=cuda), torch.zeros(16, device=cuda),
                                 torch.zeros(16, device=cuda))
    assert out.shape == (0,)


# ------------------------------------------------------------------------ config 2
def test_c2_full_vs_golden(cuda, golden):
    d = dev(inputs.c2(), cuda)
    y = ops.softmax_layernorm(d["x"], d["g"], d["gamma"], d["beta"], 1e-5)
    rows = golden["c2_rows"].tolist()
    got = y[rows].cpu()
    assert graphs.max_rel_err(got, golden["c2_y_f64"]) <= TOL_HALF
    assert graphs.max_rel_err(got, golden["c2_y_fused_f32"]) <= TOL_HALF
    assert graphs.max_rel_err(got, golden["c2_y_eager"]) <= TOL_HALF
    # size-independent properties on every row: LayerNorm output with gamma, beta removed
    # has zero mean and unit variance
    z = (y.float() - d["beta"].float()) / d["gamma"].float()
    assert float(z.mean(-1).abs().max()) < 2e-2
    assert float((z.var(-1, unbiased=False) - 1).abs().max()) < 3e-2
    # and the kernel is deterministic
    y2 = ops.softmax_layernorm(d["x"], d["g"], d["gamma"], d["beta"], 1e-5)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,cols", [(1, 8), (5, 4096), (17, 1000), (3, 4097), (9, 64), (2, 16384),
                                       (300, 768)])
def test_c2_shapes_vs_oracle(cuda, dtype, rows, cols):
    d = inputs.c2(rows, cols, seed=rows + cols, dtype=dtype)
    exp = c_oracle.softmax_layernorm(**d)
    y = ops.softmax_layernorm(**dev(d, cuda)).cpu()
    tol = 2e-5 if dtype == torch.float32 else TOL_HALF
    assert graphs.max_rel_err(y, exp) <= tol


@pytest.mark.parametrize("team,vpt", [(128, 4), (256, 2), (256, 4), (512, 2), (512, 4), (1024, 4)])
def test_c2_every_config(cuda, team, vpt):
    d = inputs.c2(64, 4096, seed=3)
    exp = graphs.softmax_layernorm(**d)
    y = ops.softmax_layernorm(**dev(d, cuda), cfg={"team": team, "vpt": vpt}).cpu()
    assert graphs.max_rel_err(y, exp) <= TOL_HALF


def test_c2_small_vs_golden(cuda, golden):
    d = inputs.c2(16, 4096, seed=12)
    y = ops.softmax_layernorm(**dev(d, cuda)).cpu()
    assert graphs.max_rel_err(y, golden["c2_small_y"]) <= TOL_HALF


# ------------------------------------------------------------------------ config 3a
def test_c3a_full_vs_golden(cuda, golden):
    x = inputs.c3a()["x"].to(cuda)
    a, b, c, dd = x.shape
    amax = ops.outer_reduce(x.view(a * b, c, dd), "amax").view(a, b, dd)
    ssum = ops.short_row_reduce(x, "sum", (c * b, 1, b)).view(a, c, b)
    slabs = golden["c3a_slabs"].tolist()
    assert torch.equal(amax[slabs].cpu(), golden["c3a_amax"])  # max is exact in fp16
    assert graphs.max_rel_err(ssum[slabs].cpu(), golden["c3a_sum_f32acc"]) <= TOL_HALF
    assert graphs.max_rel_err(ssum[slabs].cpu(), golden["c3a_sum_eager"]) <= TOL_HALF
    # whole-tensor cross-check against eager CUDA PyTorch (secondary oracle on the box)
    p = x.permute(0, 2, 1, 3)
    assert torch.equal(amax, p.amax(1))
    assert graphs.max_rel_err(ssum.cpu(), p.float().sum(3).half().cpu()) <= 2e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("kind", ["amax", "amin", "sum", "mean"])
@pytest.mark.parametrize("shape", [(3, 8, 16, 64), (2, 5, 7, 8), (1, 1, 300, 24), (4, 3, 33, 40),
                                   (2, 2, 2, 1024)])
def test_outer_reduce_shapes(cuda, dtype, kind, shape):
    a, b, c, dd = shape
    x = inputs.c3a(shape, seed=sum(shape), dtype=dtype)["x"]
    exp = c_oracle.reduce_mid(x.reshape(a * b, c, dd), kind)
    out = ops.outer_reduce(x.to(cuda).view(a * b, c, dd), kind).cpu()
    if kind in ("amax", "amin"):
        assert torch.equal(out.double(), exp)
    else:
        assert graphs.max_rel_err(out, exp) <= (TOL_F32 if dtype == torch.float32 else TOL_HALF)


@pytest.mark.parametrize("rsplit", [2, 3, 8])
@pytest.mark.parametrize("kind", ["sum", "amax"])
def test_outer_reduce_split_matches_unsplit(cuda, rsplit, kind):
    x = inputs.c3a((1, 2, 4099, 128), seed=9, dtype=torch.float32)["x"].to(cuda).view(2, 4099, 128)
    exp = c_oracle.reduce_mid(x.cpu(), kind)
    one = ops.outer_reduce(x, kind, rsplit=1).cpu()
    many = ops.outer_reduce(x, kind, rsplit=rsplit).cpu()
    assert graphs.max_rel_err(one, exp) <= TOL_F32
    assert graphs.max_rel_err(many, exp) <= TOL_F32
    if kind == "amax":
        assert torch.equal(one, many)


def test_outer_reduce_split_needs_scratch(cuda):
    x = torch.zeros(1, 1024, 64, device=cuda)
    out = torch.empty(1, 64, device=cuda)
    cfg = rt.IxbCfg(rsplit=4)
    import ctypes

    st = rt.load().ixb_outer_reduce(rt.IXB_F32, rt.IXB_SUM, x.data_ptr(), out.data_ptr(), 1, 1024, 64,
                                    None, 0, ctypes.byref(cfg), rt.raw_stream(cuda))
    assert st == rt.IXB_ERR_SCRATCH


def test_outer_reduce_nan_propagates(cuda):
    x = torch.zeros(2, 40, 16, device=cuda)
    x[1, 17, 3] = float("nan")
    out = ops.outer_reduce(x, "amax")
    assert torch.isnan(out[1, 3]) and int(torch.isnan(out).sum()) == 1


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(3, 8, 16, 64), (2, 33, 70, 8), (1, 5, 3, 128), (2, 40, 40, 16)])
@pytest.mark.parametrize("order", ["acb", "abc"])
def test_short_row_shapes(cuda, dtype, shape, order):
    a, b, c, L = shape
    x = inputs.c3a(shape, seed=sum(shape) + 1, dtype=dtype)["x"]
    s = x.double().sum(3)  # [a, b, c]
    if order == "acb":
        exp, strides = s.permute(0, 2, 1).contiguous(), (c * b, 1, b)
    else:
        exp, strides = s, (b * c, c, 1)
    out = ops.short_row_reduce(x.to(cuda), "sum", strides).view(exp.shape).cpu()
    assert graphs.max_rel_err(out, exp) <= (TOL_F32 if dtype == torch.float32 else TOL_HALF)


def test_c3a_small_vs_golden(cuda, golden):
    x = inputs.c3a((3, 8, 16, 64), seed=13)["x"].to(cuda)
    amax = ops.outer_reduce(x.view(24, 16, 64), "amax").view(3, 8, 64).cpu()
    ssum = ops.short_row_reduce(x, "sum", (16 * 8, 1, 8)).view(3, 16, 8).cpu()
    assert torch.equal(amax, golden["c3a_small_amax"])
    assert graphs.max_rel_err(ssum, golden["c3a_small_sum"]) <= TOL_HALF


# ------------------------------------------------------------------------ config 3b
def test_c3b_full_bit_exact(cuda, golden):
    d = inputs.c3b()
    out = ops.index_select_rows(d["table"].to(cuda), d["idx"].to(cuda)).cpu()
    assert torch.equal(out[:8], golden["c3b_head"])
    assert hashlib.sha256(out.view(torch.uint8).numpy().tobytes()).hexdigest() == golden["c3b_sha256"]


@pytest.mark.parametrize("dtype,dim", [(torch.float16, 128), (torch.float32, 3), (torch.bfloat16, 7),
                                       (torch.int64, 2), (torch.uint8, 5), (torch.float32, 1000),
                                       (torch.float16, 8)])
@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_gather_shapes_bit_exact(cuda, dtype, dim, idx_dtype):
    g = torch.Generator().manual_seed(dim)
    table = torch.randint(0, 255, (97, dim), generator=g).to(dtype)
    idx = torch.randint(0, 97, (1001,), generator=g, dtype=torch.int64)
    exp, bad = c_oracle.index_select_rows(table, idx)
    assert bad == 0
    out = ops.index_select_rows(table.to(cuda), idx.to(idx_dtype).to(cuda)).cpu()
    assert torch.equal(out, exp) and torch.equal(out, table.index_select(0, idx))


def test_gather_edge_cases(cuda):
    table = torch.arange(40, dtype=torch.float32, device=cuda).reshape(10, 4)
    empty = ops.index_select_rows(table, torch.empty(0, dtype=torch.int64, device=cuda))
    assert empty.shape == (0, 4)
    neg = ops.index_select_rows(table, torch.tensor([-1, 0, -10], device=cuda), wrap_negative=True)
    assert torch.equal(neg.cpu(), table.cpu()[[9, 0, 0]])
    with pytest.raises(IndexError):
        ops.index_select_rows(table, torch.tensor([0, 10], device=cuda))
    with pytest.raises(IndexError):
        ops.index_select_rows(table, torch.tensor([-1], device=cuda))
    # the context is still usable and the bad row is zero-filled when unchecked
    out = ops.index_select_rows(table, torch.tensor([3, 11], device=cuda), check_bounds=False)
    assert torch.equal(out.cpu(), torch.stack([table[3].cpu(), torch.zeros(4)]))
    # strided table (row pitch > row bytes)
    wide = torch.arange(80, dtype=torch.float32, device=cuda).reshape(10, 8)
    view = wide[:, :4]
    got = ops.index_select_rows(view, torch.tensor([9, 2], device=cuda))
    assert torch.equal(got, view[[9, 2]])


# ------------------------------------------------------------------ generic row ops
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("kind", ["sum", "mean", "amax", "amin", "argmax", "argmin", "var_mean"])
@pytest.mark.parametrize("shape", [(8, 16, 64), (13, 1023), (2053, 9), (4, 4096), (3, 20000)])
def test_row_reduce(cuda, dtype, kind, shape):
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(*shape, generator=g).to(dtype)
    xd = x.double()
    res = ops.row_reduce(x.to(cuda), kind)
    tol = TOL_F32 * 4 if dtype == torch.float32 else TOL_HALF
    if kind in ("argmax", "argmin"):
        exp = getattr(x.float(), kind)(-1)
        assert torch.equal(res.cpu(), exp)
    elif kind in ("amax", "amin"):
        assert torch.equal(res.cpu(), getattr(x, kind)(-1))
    elif kind == "var_mean":
        var, mean = res
        ev, em = torch.var_mean(xd, -1, correction=1)
        assert graphs.max_rel_err(var.cpu(), ev) <= tol
        assert graphs.max_rel_err(mean.cpu(), em, floor=1.0 / shape[-1] ** 0.5) <= tol
    else:
        exp = getattr(xd, kind)(-1)
        floor = float(exp.abs().mean()) or 1.0
        assert graphs.max_rel_err(res.cpu(), exp, floor=floor) <= tol


def test_argmax_ties_and_nan(cuda):
    x = torch.zeros(3, 700, device=cuda)
    x[0, 5] = x[0, 600] = 2.0
    x[1, 650] = float("nan")
    x[1, 3] = 9.0
    assert ops.row_reduce(x, "argmax").tolist() == torch.argmax(x.cpu(), -1).tolist()
    assert ops.row_reduce(x, "argmin").tolist() == torch.argmin(x.cpu(), -1).tolist()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,cols", [(9, 4096), (4, 1000), (100, 128)])
def test_rmsnorm(cuda, dtype, rows, cols):
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, cols, generator=g).to(dtype)
    r = torch.randn(rows, cols, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
    y = ops.rmsnorm(x.to(cuda), w.to(cuda), 1e-6).cpu()
    assert graphs.max_rel_err(y, graphs.rmsnorm(x, w, 1e-6, torch.float64)) <= TOL_HALF
    y2, h = ops.rmsnorm(x.to(cuda), w.to(cuda), 1e-6, residual=r.to(cuda), return_residual=True)
    ey, eh = graphs.add_rmsnorm(x, r, w, 1e-6, torch.float64)
    assert torch.equal(h.cpu(), eh)
    assert graphs.max_rel_err(y2.cpu(), ey) <= TOL_HALF


def test_host_row_pipeline_matches_direct_call(cuda):
    from inductor_x_b200.host_io import HostRowPipeline

    d = inputs.c2(1000, 4096, seed=31)
    params = [d[k].to(cuda) for k in ("g", "gamma", "beta")]
    h_x = d["x"].pin_memory()
    h_y = torch.empty_like(h_x).pin_memory()
    pipe = HostRowPipeline(cuda, h_x.shape, h_x.dtype, h_x.shape, h_x.dtype, chunks=7)
    for _ in range(2):  # second call reuses the staging buffers
        pipe.run(h_x, lambda xc, out: ops.softmax_layernorm(xc, *params, 1e-5, out=out), h_y)
        torch.cuda.synchronize()
        direct = ops.softmax_layernorm(d["x"].to(cuda), *params, 1e-5).cpu()
        assert torch.equal(h_y, direct)
