"""ctypes binding of the C restatement (``ixb_oracle.c``).  Test infrastructure only."""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import c_double, c_int, c_int64, c_void_p

import numpy as np
import torch

_DIR = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_DIR, "_build", "libixb_oracle.so")
_lib = None


def build() -> str:
    subprocess.run(["make", "-C", _DIR], check=True, capture_output=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.orc_index_select_rows.restype = c_int64
    return _lib


def _f32(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.detach().to(torch.float32).cpu().numpy())


def _p(a: np.ndarray):
    return a.ctypes.data_as(c_void_p)


def affine_gelu_rowsum(x, w, b) -> torch.Tensor:
    xa, wa, ba = _f32(x), _f32(w), _f32(b)
    rows, cols = xa.shape
    out = np.empty(rows, dtype=np.float64)
    lib().orc_affine_gelu_rowsum(_p(xa), _p(wa), _p(ba), _p(out), c_int64(rows), c_int64(cols))
    return torch.from_numpy(out)


def softmax_layernorm(x, g, gamma, beta, eps=1e-5) -> torch.Tensor:
    xa, ga, gm, be = _f32(x), _f32(g), _f32(gamma), _f32(beta)
    cols = xa.shape[-1]
    rows = xa.size // cols
    y = np.empty(xa.shape, dtype=np.float64)
    lib().orc_softmax_layernorm(_p(xa), _p(ga), _p(gm), _p(be), _p(y), c_int64(rows), c_int64(cols),
                                c_double(eps))
    return torch.from_numpy(y)


def reduce_mid(x, kind: str) -> torch.Tensor:
    xa = _f32(x)
    outer, R, inner = xa.shape
    out = np.empty((outer, inner), dtype=np.float64)
    code = {"sum": 0, "mean": 1, "amax": 2, "amin": 3}[kind]
    lib().orc_reduce_mid(_p(xa), _p(out), c_int64(outer), c_int64(R), c_int64(inner), c_int(code))
    return torch.from_numpy(out)


def index_select_rows(table: torch.Tensor, idx: torch.Tensor, wrap_negative=False):
    """Returns (rows as a tensor of table's dtype, position+1 of first bad index or 0)."""
    t = table.detach().cpu().contiguous()
    raw = t.view(torch.uint8).numpy() if t.dtype != torch.bfloat16 else t.view(torch.int16).numpy().view(np.uint8)
    n_rows = t.shape[0]
    row_bytes = t[0].numel() * t.element_size() if n_rows else 0
    ia = np.ascontiguousarray(idx.detach().cpu().to(torch.int64).numpy())
    out = np.empty((ia.size, row_bytes), dtype=np.uint8)
    bad = lib().orc_index_select_rows(_p(np.ascontiguousarray(raw)), _p(ia), _p(out), c_int64(n_rows),
                                      c_int64(ia.size), c_int64(row_bytes), c_int(int(wrap_negative)))
    res = torch.from_numpy(out).view(t.dtype).reshape(ia.size, *t.shape[1:])
    return res, int(bad)


def attention(q, k, v, scale, causal=True):
    """[B, H, S, D] attention in double; returns (out fp64, lse fp64)."""
    qa, ka, va = _f32(q), _f32(k), _f32(v)
    B, H, Sq, D = qa.shape
    Sk = ka.shape[2]
    out = np.empty((B, H, Sq, D), dtype=np.float64)
    lse = np.empty((B, H, Sq), dtype=np.float64)
    for b in range(B):
        for h in range(H):
            lib().orc_attention_head(_p(qa[b, h]), _p(ka[b, h]), _p(va[b, h]), _p(out[b, h]),
                                     _p(lse[b, h]), c_int64(Sq), c_int64(Sk), c_int64(D),
                                     c_double(scale), c_int(int(causal)))
    return torch.from_numpy(out), torch.from_numpy(lse)
