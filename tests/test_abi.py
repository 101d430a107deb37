"""CPU tests of the boundary: the shared library loads, exports exactly the symbols the
header declares, and its host-side logic (error strings, launch chooser) behaves."""
import ctypes
import os
import re

import pytest
import torch

from inductor_x_b200 import runtime as rt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names += re.findall(r"\b(ixb_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_loads_and_exports_every_declared_symbol():
    lib = rt.load()
    syms = header_symbols()
    assert len(syms) >= 10
    for name in syms:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    # and the Python binding table covers the same set
    assert sorted(rt.declared_symbols()) == syms


def test_abi_version_and_strerror():
    lib = rt.load()
    assert lib.ixb_abi_version() == 1
    assert lib.ixb_strerror(0) == b"ok"
    for code in range(1, 9):
        assert lib.ixb_strerror(code) not in (b"ok", b"unknown status")
    assert lib.ixb_strerror(99) == b"unknown status"


def test_argument_validation_needs_no_gpu():
    lib = rt.load()
    # null pointers / bad sizes are rejected before any CUDA call
    assert lib.ixb_affine_gelu_rowsum_f32(None, None, None, None, 4, 8, None, None) == rt.IXB_ERR_ARG
    assert lib.ixb_affine_gelu_rowsum_f32(None, None, None, None, 0, 8, None, None) == rt.IXB_OK
    assert lib.ixb_softmax_layernorm(rt.IXB_BF16, None, None, None, None, None, -1, 8, 0.0, None, None) == rt.IXB_ERR_ARG
    assert lib.ixb_row_reduce(rt.IXB_F32, rt.IXB_SUM, None, None, None, 0, 8, 0.0, None, None) == rt.IXB_OK
    assert lib.ixb_index_select_rows(None, None, None, 4, 0, 16, 16, rt.IXB_I64, 0, None, None) == rt.IXB_OK
    assert lib.ixb_index_select_rows(None, None, None, 4, 2, 16, 8, rt.IXB_I64, 0, None, None) == rt.IXB_ERR_ARG
    assert lib.ixb_outer_reduce_scratch_bytes(10, 20, 1) == 0
    assert lib.ixb_outer_reduce_scratch_bytes(10, 20, 4) == 10 * 20 * 4 * 4


@pytest.mark.parametrize("dtype,cols,team,vpt", [
    (torch.bfloat16, 4096, 128, 4),
    (torch.float32, 1024, 64, 4),
    (torch.float16, 64, 32, 1),
    (torch.float32, 1023, 64, 4),
    (torch.bfloat16, 65536, 1024, 8),
])
def test_row_chooser(dtype, cols, team, vpt):
    cfg = rt.choose_config(rt.IXB_FAM_ROW, dtype, 1000, cols)
    assert (cfg.team, cfg.vpt) == (team, vpt)
    vec = 16 // torch.empty(0, dtype=dtype).element_size()
    assert cfg.team * cfg.vpt * vec >= cols


def test_row_chooser_rejects_oversized_rows():
    with pytest.raises(rt.IxbError) as e:
        rt.choose_config(rt.IXB_FAM_ROW, torch.float32, 10, 1 << 20)
    assert e.value.status == rt.IXB_ERR_SHAPE


def test_outer_chooser_split_factor():
    # plenty of kept extent: no split
    assert rt.choose_config(rt.IXB_FAM_OUTER, torch.float16, 8192, 256, 64).rsplit == 1
    # tiny kept extent, long reduced axis: split so that >= 2 waves of CTAs exist
    cfg = rt.choose_config(rt.IXB_FAM_OUTER, torch.float32, 1, 1 << 16, 128)
    assert cfg.rsplit > 1 and (1 << 16) // cfg.rsplit >= 256
    dev = rt.IxbDevInfo(sm_count=148)
    assert rt.choose_config(rt.IXB_FAM_OUTER, torch.float32, 1, 1 << 16, 128, dev=dev).rsplit == cfg.rsplit


def test_ops_reject_cpu_tensors():
    from inductor_x_b200 import ops

    x = torch.zeros(4, 8)
    with pytest.raises(ValueError):
        ops.affine_gelu_rowsum(x, torch.zeros(8), torch.zeros(8))
    with pytest.raises(ValueError):
        ops.index_select_rows(x, torch.zeros(2, dtype=torch.int64))
