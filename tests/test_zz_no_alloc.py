"""GPU test of ixb_outer_reduce_static, the entry point that allocates nothing.

Some callers cannot give the library scratch memory: generated wrappers whose buffers
were all planned up front, serving loops where a cudaMalloc would stall the device, or
processes whose GPU memory already belongs to a caching allocator.  For them the split
outer reduction keeps its partial sums in a fixed array inside the library.  The test
calls it twice in a row through the C ABI (the array is shared by every call and keeps
the previous call's contents) and compares with the ordinary entry point, which takes
caller-provided scratch.  Collected last so that a failure here cannot mask other tests.
"""
import ctypes

import pytest
import torch

from inductor_x_b200 import ops
from inductor_x_b200 import runtime as rt
from oracle import c_oracle, graphs

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5
TOL_HALF = 2e-2


def call_static(x, kind, rsplit):
    outer, R, inner = x.shape
    out = torch.empty(outer, inner, dtype=x.dtype, device=x.device)
    st = rt.load().ixb_outer_reduce_static(rt.DTYPE_CODE[x.dtype], rt.REDUCE_CODE[kind], x.data_ptr(),
                                           out.data_ptr(), outer, R, inner, rsplit,
                                           rt.raw_stream(x.device))
    return st, out


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_F32), (torch.bfloat16, TOL_HALF)])
def test_static_scratch_matches_caller_scratch_twice(cuda, dtype, tol):
    g = torch.Generator().manual_seed(7)
    # two different problems back to back: the second must not see the first's partials
    xa = torch.randn(2, 4099, 128, generator=g).to(dtype).to(cuda)
    xb = (torch.randn(3, 2048, 64, generator=g) * 3 + 1).to(dtype).to(cuda)
    for x, kind, rsplit in ((xa, "sum", 8), (xb, "amax", 4), (xa, "mean", 3)):
        st, got = call_static(x, kind, rsplit)
        assert st == rt.IXB_OK, rt.load().ixb_strerror(st)
        ref = ops.outer_reduce(x, kind, rsplit=rsplit)
        assert graphs.max_rel_err(got.cpu(), ref.cpu()) <= tol
        exp = c_oracle.reduce_mid(x.cpu(), kind)
        if kind == "amax":
            assert torch.equal(got.cpu().double(), exp)
        else:
            assert graphs.max_rel_err(got.cpu(), exp) <= tol


def test_static_scratch_rejects_oversize_and_misuse(cuda):
    lib = rt.load()
    x = torch.zeros(1, 1024, 4096, device=cuda)
    # 1 * 4096 * 512 floats = 8 MiB of partials: over the 4 MiB array
    st, _ = call_static(x, "sum", 512)
    assert st == rt.IXB_ERR_SCRATCH
    assert b"scratch" in lib.ixb_strerror(st)
    st, _ = call_static(x, "sum", 256)  # exactly 4 MiB fits
    assert st == rt.IXB_OK
    odd = torch.zeros(2, 64, 6, device=cuda)  # inner not a multiple of 16 bytes
    st, _ = call_static(odd, "sum", 2)
    assert st == rt.IXB_ERR_ALIGN
    st, _ = call_static(x, "sum", 0)
    assert st == rt.IXB_ERR_ARG
    torch.cuda.synchronize()
