"""ctypes binding of ``libixb.so`` - the C ABI declared in ``include/ixb.h``.

This module is the only place Python touches the native library.  It plays the part of
the launcher closure the reference builds per compiled kernel
(``inductor_x/npu_triton_heuristics.py:239-253``: ``launcher(*args, grid, stream)``) and
of ``get_current_raw_stream`` (``inductor_x/__init__.py:26-27``).

There is deliberately no fallback: if the library is missing or a call fails, an
exception is raised.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from typing import Optional

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# IXB_LIB_PATH points at an alternative build of the library (e.g. an instrumented one)
LIB_PATH = os.environ.get("IXB_LIB_PATH") or os.path.join(_PKG_DIR, "libixb.so")

IXB_OK = 0
IXB_ERR_ARG, IXB_ERR_DTYPE, IXB_ERR_ALIGN, IXB_ERR_SHAPE = 1, 2, 3, 4
IXB_ERR_UNSUPPORTED, IXB_ERR_SCRATCH, IXB_ERR_CUDA, IXB_ERR_INDEX = 5, 6, 7, 8

IXB_F32, IXB_F16, IXB_BF16, IXB_I64, IXB_I32, IXB_U8 = 0, 1, 2, 3, 4, 5
IXB_SUM, IXB_MEAN, IXB_AMAX, IXB_AMIN, IXB_ARGMAX, IXB_ARGMIN, IXB_VAR_MEAN = range(7)
(IXB_FAM_POINTWISE, IXB_FAM_ROW, IXB_FAM_OUTER, IXB_FAM_SHORT_ROW, IXB_FAM_GATHER) = range(5)

DTYPE_CODE = {
    torch.float32: IXB_F32,
    torch.float16: IXB_F16,
    torch.bfloat16: IXB_BF16,
    torch.int64: IXB_I64,
    torch.int32: IXB_I32,
    torch.uint8: IXB_U8,
}
REDUCE_CODE = {
    "sum": IXB_SUM, "mean": IXB_MEAN, "amax": IXB_AMAX, "max": IXB_AMAX, "amin": IXB_AMIN,
    "min": IXB_AMIN, "argmax": IXB_ARGMAX, "argmin": IXB_ARGMIN, "var_mean": IXB_VAR_MEAN,
}


class IxbDevInfo(ctypes.Structure):
    _fields_ = [
        ("sm_count", c_int32), ("cc_major", c_int32), ("cc_minor", c_int32),
        ("max_threads_per_sm", c_int32), ("l2_bytes", c_int64),
        ("smem_per_block_optin", c_int64), ("global_mem_bytes", c_int64),
        ("vector_bytes", c_int32), ("reserved", c_int32),
    ]


class IxbCfg(ctypes.Structure):
    _fields_ = [
        ("team", c_int32), ("vpt", c_int32), ("grid", c_int32), ("rsplit", c_int32),
        ("threads", c_int32), ("unroll", c_int32), ("reserved", c_int32 * 2),
    ]

    def as_dict(self):
        return {k: getattr(self, k) for k in ("team", "vpt", "grid", "rsplit", "threads", "unroll")}


class IxbProblem(ctypes.Structure):
    _fields_ = [
        ("family", c_int32), ("dtype", c_int32), ("outer", c_int64), ("reduce", c_int64),
        ("inner", c_int64), ("row_inputs", c_int32), ("aligned", c_int32),
    ]


class IxbError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, status: int, detail: str):
        super().__init__(f"{fn} failed: status {status} ({detail})")
        self.status = status


# name -> (restype, argtypes); every symbol include/ixb.h declares is listed here and
# tests check the two stay in step.
_SIGNATURES = {
    "ixb_abi_version": (c_int, []),
    "ixb_strerror": (c_char_p, [c_int]),
    "ixb_last_cuda_error": (c_char_p, []),
    "ixb_device_info": (c_int, [c_int, POINTER(IxbDevInfo)]),
    "ixb_choose_config": (c_int, [POINTER(IxbProblem), POINTER(IxbDevInfo), POINTER(IxbCfg)]),
    "ixb_affine_gelu_rowsum_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                           POINTER(IxbCfg), c_void_p]),
    "ixb_softmax_layernorm": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                      c_int64, c_float, POINTER(IxbCfg), c_void_p]),
    "ixb_rmsnorm": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                            c_float, POINTER(IxbCfg), c_void_p]),
    "ixb_row_reduce": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float,
                               POINTER(IxbCfg), c_void_p]),
    "ixb_outer_reduce_scratch_bytes": (c_size_t, [c_int64, c_int64, c_int]),
    "ixb_outer_reduce": (c_int, [c_int, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p,
                                 c_size_t, POINTER(IxbCfg), c_void_p]),
    "ixb_outer_reduce_static": (c_int, [c_int, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                                        c_void_p]),
    "ixb_short_row_reduce": (c_int, [c_int, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                     c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "ixb_fa_fwd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32,
                           c_int32, c_int32, c_int32, POINTER(c_int64), POINTER(c_int64),
                           POINTER(c_int64), POINTER(c_int64), c_float, c_int, c_void_p, c_void_p]),
    "ixb_fa_bwd": (c_int, [c_int] + [c_void_p] * 10 + [c_int32] * 5 + [POINTER(c_int64)] * 8 +
                   [c_float, c_int, c_void_p, c_void_p]),
    "ixb_index_select_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                      c_int, c_int, c_void_p, c_void_p]),
    "ixb_cp_forward_update": (c_int, [c_int] + [c_void_p] * 9 + [c_int32] * 4 + [c_int64] * 3 + [c_void_p]),
    "ixb_cp_forward_update_lse": (c_int, [c_void_p] * 4 + [c_int32] * 4 + [c_int64] * 4 + [c_void_p]),
    "ixb_cp_accumulate": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_void_p]),
}

_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Load ``libixb.so`` (once) and bind every declared symbol.  Raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `make -C {os.path.join(_PKG_DIR, 'csrc')}` "
            "(or __graft_entry__.build()); this backend has no non-CUDA path")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.ixb_abi_version() != 1:
        raise ImportError(f"{LIB_PATH}: ABI version {lib.ixb_abi_version()} != 1")
    _lib = lib
    return lib


def declared_symbols():
    return list(_SIGNATURES)


#: kernel-launching entry points of the library called successfully by this process
native_calls = 0


def check(fn: str, status: int) -> None:
    global native_calls
    native_calls += 1
    if status != IXB_OK:
        lib = load()
        detail = lib.ixb_strerror(status).decode()
        if status == IXB_ERR_CUDA:
            detail += ": " + lib.ixb_last_cuda_error().decode()
        raise IxbError(fn, status, detail)


def raw_stream(device=None) -> int:
    """Handle of the current CUDA stream of ``device`` (the reference's
    ``get_current_raw_stream``, ``inductor_x/__init__.py:26-27``)."""
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def make_cfg(cfg) -> Optional[IxbCfg]:
    """None, an IxbCfg or a dict of IxbCfg fields."""
    if cfg is None or isinstance(cfg, IxbCfg):
        return cfg
    c = IxbCfg()
    for k, v in dict(cfg).items():
        setattr(c, k, int(v))
    return c


def device_info(device: int = -1) -> IxbDevInfo:
    info = IxbDevInfo()
    check("ixb_device_info", load().ixb_device_info(device, ctypes.byref(info)))
    return info


def choose_config(family: int, dtype: torch.dtype, outer: int, reduce: int, inner: int = 0,
                  row_inputs: int = 1, aligned: bool = True,
                  dev: Optional[IxbDevInfo] = None) -> IxbCfg:
    """Launch configuration the library would pick (host arithmetic; no GPU needed when
    ``dev`` is given or left None, in which case B200 defaults apply)."""
    pb = IxbProblem(family, DTYPE_CODE[dtype], outer, reduce, inner, row_inputs, int(aligned))
    cfg = IxbCfg()
    devp = ctypes.byref(dev) if dev is not None else None
    check("ixb_choose_config", load().ixb_choose_config(ctypes.byref(pb), devp, ctypes.byref(cfg)))
    return cfg
