"""Tensor-level entry points over the C ABI: one function per prebuilt kernel family.

These are what the generated wrapper code, the tests and ``bench.py`` call.  Each takes
CUDA tensors, validates layout, allocates the output with torch (plumbing only) and
enqueues exactly the native kernels on the current stream.  A CPU tensor is rejected:
there is no host path.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch

from . import runtime as rt


def launch_count() -> int:
    """Calls made into the kernel library's launching entry points so far (each enqueues one
    kernel; a split outer reduction two)."""
    return rt.native_calls


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("inductor_x_b200 kernels take CUDA tensors only (no CPU path)")


def _cfg_ref(cfg):
    c = rt.make_cfg(cfg)
    return (ctypes.byref(c) if c is not None else None), c


def affine_gelu_rowsum(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, *, out=None, cfg=None):
    """``sum(gelu(x * w + b), dim=-1)`` for fp32 ``x[rows, cols]``, ``w[cols]``, ``b[cols]``."""
    _need_cuda(x, w, b)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise ValueError("x must be a contiguous fp32 matrix")
    rows, cols = x.shape
    if w.shape != (cols,) or b.shape != (cols,) or w.dtype != x.dtype or b.dtype != x.dtype:
        raise ValueError("w and b must be fp32 vectors of length cols")
    w, b = w.contiguous(), b.contiguous()
    if out is None:
        out = torch.empty(rows, dtype=x.dtype, device=x.device)
    ref, keep = _cfg_ref(cfg)
    rt.check("ixb_affine_gelu_rowsum_f32", rt.load().ixb_affine_gelu_rowsum_f32(
        x.data_ptr(), w.data_ptr(), b.data_ptr(), out.data_ptr(), rows, cols, ref,
        rt.raw_stream(x.device)))
    return out


def softmax_layernorm(x, g, gamma, beta, eps: float = 1e-5, *, out=None, cfg=None):
    """``layer_norm(softmax(x, -1) * g + x, [cols], gamma, beta, eps)`` in one pass."""
    _need_cuda(x, g, gamma, beta)
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"unsupported dtype {x.dtype}")
    if not x.is_contiguous() or x.dim() < 1:
        raise ValueError("x must be contiguous")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    for name, v in (("g", g), ("gamma", gamma), ("beta", beta)):
        if v.shape != (cols,) or v.dtype != x.dtype:
            raise ValueError(f"{name} must have shape ({cols},) and dtype {x.dtype}")
    g, gamma, beta = g.contiguous(), gamma.contiguous(), beta.contiguous()
    if out is None:
        out = torch.empty_like(x)
    ref, keep = _cfg_ref(cfg)
    rt.check("ixb_softmax_layernorm", rt.load().ixb_softmax_layernorm(
        rt.DTYPE_CODE[x.dtype], x.data_ptr(), g.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
        out.data_ptr(), rows, cols, float(eps), ref, rt.raw_stream(x.device)))
    return out


def rmsnorm(x, w, eps: float = 1e-6, *, residual=None, return_residual: bool = False, cfg=None):
    """RMSNorm over the last axis with an optional fused residual add.

    Returns ``y`` or ``(y, h)`` where ``h = x + residual`` (rounded to the storage dtype)."""
    _need_cuda(x, w, residual)
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    if w.shape != (cols,) or w.dtype != x.dtype:
        raise ValueError("w must be a vector of length cols in x's dtype")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype
                                 or not residual.is_contiguous()):
        raise ValueError("residual must match x")
    y = torch.empty_like(x)
    h = torch.empty_like(x) if (residual is not None and return_residual) else None
    ref, keep = _cfg_ref(cfg)
    rt.check("ixb_rmsnorm", rt.load().ixb_rmsnorm(
        rt.DTYPE_CODE[x.dtype], x.data_ptr(), rt.ptr(residual), w.contiguous().data_ptr(),
        y.data_ptr(), rt.ptr(h), rows, cols, float(eps), ref, rt.raw_stream(x.device)))
    return (y, h) if h is not None else y


def row_reduce(x: torch.Tensor, kind: str, *, correction: float = 1.0, cfg=None):
    """Reduce the last axis of contiguous ``x``.  ``kind``: sum, mean, amax, amin, argmax,
    argmin or var_mean (returns ``(var, mean)``)."""
    _need_cuda(x)
    if not x.is_contiguous() or x.dim() < 1:
        raise ValueError("x must be contiguous")
    code = rt.REDUCE_CODE[kind]
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    lead = x.shape[:-1]
    out_dtype = torch.int64 if code in (rt.IXB_ARGMAX, rt.IXB_ARGMIN) else x.dtype
    out = torch.empty(lead, dtype=out_dtype, device=x.device)
    out2 = torch.empty(lead, dtype=x.dtype, device=x.device) if code == rt.IXB_VAR_MEAN else None
    ref, keep = _cfg_ref(cfg)
    rt.check("ixb_row_reduce", rt.load().ixb_row_reduce(
        rt.DTYPE_CODE[x.dtype], code, x.data_ptr(), out.data_ptr(), rt.ptr(out2), rows, cols,
        float(correction), ref, rt.raw_stream(x.device)))
    return (out, out2) if out2 is not None else out


def outer_reduce(x: torch.Tensor, kind: str, *, rsplit: int = 0, scratch: Optional[torch.Tensor] = None):
    """Reduce the middle axis of contiguous ``x[outer, R, inner]`` -> ``[outer, inner]``.

    ``rsplit`` > 1 forces a split of the reduced axis (0 = library's choice); the fp32
    scratch it needs is taken from ``scratch`` or allocated here with torch."""
    _need_cuda(x, scratch)
    if x.dim() != 3 or not x.is_contiguous():
        raise ValueError("x must be a contiguous [outer, R, inner] tensor")
    outer, R, inner = x.shape
    code = rt.REDUCE_CODE[kind]
    lib = rt.load()
    if rsplit <= 0 and outer and inner:
        rsplit = rt.choose_config(rt.IXB_FAM_OUTER, x.dtype, outer, R, inner).rsplit
    need = lib.ixb_outer_reduce_scratch_bytes(outer, inner, rsplit)
    if need and (scratch is None or scratch.numel() * scratch.element_size() < need):
        scratch = torch.empty(need // 4, dtype=torch.float32, device=x.device)
    out = torch.empty((outer, inner), dtype=x.dtype, device=x.device)
    cfg = rt.IxbCfg(rsplit=max(rsplit, 1))
    sbytes = scratch.numel() * scratch.element_size() if scratch is not None else 0
    rt.check("ixb_outer_reduce", lib.ixb_outer_reduce(
        rt.DTYPE_CODE[x.dtype], code, x.data_ptr(), out.data_ptr(), outer, R, inner, rt.ptr(scratch),
        sbytes, ctypes.byref(cfg), rt.raw_stream(x.device)))
    return out


def short_row_reduce(x: torch.Tensor, kind: str, out_strides: Sequence[int],
                     out: Optional[torch.Tensor] = None):
    """Reduce the short stride-1 axis of contiguous ``x[A, B, C, L]`` and store result
    ``(a, b, c)`` at element offset ``a*sa + b*sb + c*sc`` of ``out``."""
    _need_cuda(x, out)
    if x.dim() != 4 or not x.is_contiguous():
        raise ValueError("x must be a contiguous [A, B, C, L] tensor")
    A, B, C, L = x.shape
    sa, sb, sc = (int(s) for s in out_strides)
    if out is None:
        out = torch.empty(A * B * C, dtype=x.dtype, device=x.device)
    rt.check("ixb_short_row_reduce", rt.load().ixb_short_row_reduce(
        rt.DTYPE_CODE[x.dtype], rt.REDUCE_CODE[kind], x.data_ptr(), out.data_ptr(), A, B, C, L,
        sa, sb, sc, rt.raw_stream(x.device)))
    return out


def index_select_rows(table: torch.Tensor, idx: torch.Tensor, *, wrap_negative: bool = False,
                      check_bounds: bool = True):
    """``table.index_select(0, idx)`` for a 2-D+ table whose rows are contiguous.

    With ``check_bounds`` an out-of-range index raises ``IndexError`` (this reads a device
    status word back, i.e. synchronises; pass False inside latency-critical code)."""
    _need_cuda(table, idx)
    if table.dim() < 1 or idx.dim() != 1 or idx.dtype not in (torch.int64, torch.int32):
        raise ValueError("table must have >= 1 dim, idx must be a 1-D int32/int64 tensor")
    n_rows = table.shape[0]
    row_shape = table.shape[1:]
    if table.dim() > 1 and not table[0].is_contiguous():
        raise ValueError("rows of table must be contiguous")
    row_elems = 1
    for s in row_shape:
        row_elems *= s
    row_bytes = row_elems * table.element_size()
    pitch = (table.stride(0) if table.dim() > 1 else 1) * table.element_size()
    if n_rows <= 1:
        pitch = max(pitch, row_bytes)
    idx = idx.contiguous()
    m = idx.numel()
    out = torch.empty((m, *row_shape), dtype=table.dtype, device=table.device)
    status = torch.zeros(2, dtype=torch.int32, device=table.device) if check_bounds else None
    rt.check("ixb_index_select_rows", rt.load().ixb_index_select_rows(
        table.data_ptr(), idx.data_ptr(), out.data_ptr(), n_rows, m, row_bytes, pitch,
        rt.DTYPE_CODE[idx.dtype], int(wrap_negative), rt.ptr(status), rt.raw_stream(table.device)))
    if status is not None:
        flag, pos = status.tolist()
        if flag:
            raise IndexError(f"index_select_rows: index out of range at position {pos}")
    return out


def _bhs_strides(t: torch.Tensor):
    arr = (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    return arr


def fused_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, *,
                    causal: bool = False, return_lse: bool = False, check: bool = False):
    """``softmax(q @ k^T * scale [+ causal mask]) @ v`` for ``[B, H, S, D]`` tensors
    (any batch/head/sequence strides, ``D`` contiguous, ``D == 128``, fp16 or bf16).

    Returns ``out`` (contiguous ``[B, H, Sq, D]``) or ``(out, lse)`` with ``lse`` the fp32
    log-sum-exp of the scaled scores ``[B, H, Sq]``.  ``check=True`` reads the kernel's
    status word back (synchronises) and raises if an internal wait gave up."""
    _need_cuda(q, k, v)
    if q.dim() != 4 or k.shape != v.shape or q.shape[:2] != k.shape[:2] or q.shape[3] != k.shape[3]:
        raise ValueError("expected q[B,H,Sq,D], k[B,H,Sk,D], v[B,H,Sk,D]")
    if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must share dtype float16 or bfloat16")
    for t in (q, k, v):
        if t.stride(3) != 1:
            raise ValueError("the head dimension must be contiguous")
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    out = torch.empty((B, H, Sq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device) if return_lse else None
    status = torch.zeros(1, dtype=torch.int32, device=q.device) if check else None
    rt.check("ixb_fa_fwd", rt.load().ixb_fa_fwd(
        rt.DTYPE_CODE[q.dtype], q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), rt.ptr(lse),
        B, H, Sq, Sk, D, _bhs_strides(q), _bhs_strides(k), _bhs_strides(v), _bhs_strides(out),
        float(scale), int(causal), rt.ptr(status), rt.raw_stream(q.device)))
    if status is not None and int(status.item()) != 0:
        raise RuntimeError("ixb_fa_fwd: an internal pipeline wait gave up; output is undefined")
    return (out, lse) if return_lse else out


def fused_attention_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                             lse: torch.Tensor, dout: torch.Tensor, scale: float, *, causal: bool = False,
                             check: bool = False):
    """Gradients ``(dq, dk, dv)`` of :func:`fused_attention` from its inputs, its output
    ``out``, its log-sum-exp ``lse`` (``return_lse=True``) and the incoming gradient ``dout``
    (tcgen05 kernels behind ``ixb_fa_bwd``; deterministic, no atomics)."""
    _need_cuda(q, k, v, out, dout, lse)
    if q.dim() != 4 or k.shape != v.shape or q.shape[:2] != k.shape[:2] or q.shape[3] != k.shape[3]:
        raise ValueError("expected q[B,H,Sq,D], k[B,H,Sk,D], v[B,H,Sk,D]")
    if out.shape != q.shape or dout.shape != q.shape:
        raise ValueError("out and dout must have the shape of q")
    if q.dtype not in (torch.float16, torch.bfloat16) or any(t.dtype != q.dtype for t in (k, v, out, dout)):
        raise ValueError("q, k, v, out, dout must share dtype float16 or bfloat16")
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    if lse.shape != (B, H, Sq) or lse.dtype != torch.float32:
        raise ValueError("lse must be float32 [B, H, Sq]")
    lse = lse.contiguous()
    if dout.stride(3) != 1 or any(st % 8 for st in dout.stride()[:3]):
        dout = dout.contiguous()
    for t in (q, k, v, out, dout):
        if t.stride(3) != 1:
            raise ValueError("the head dimension must be contiguous")
    dq = torch.empty((B, H, Sq, D), dtype=q.dtype, device=q.device)
    dk = torch.empty((B, H, Sk, D), dtype=q.dtype, device=q.device)
    dv = torch.empty((B, H, Sk, D), dtype=q.dtype, device=q.device)
    delta = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    status = torch.zeros(1, dtype=torch.int32, device=q.device) if check else None
    rt.check("ixb_fa_bwd", rt.load().ixb_fa_bwd(
        rt.DTYPE_CODE[q.dtype], q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
        lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr(), B, H, Sq, Sk, D,
        _bhs_strides(q), _bhs_strides(k), _bhs_strides(v), _bhs_strides(out), _bhs_strides(dout),
        _bhs_strides(dq), _bhs_strides(dk), _bhs_strides(dv), float(scale), int(causal), rt.ptr(status),
        rt.raw_stream(q.device)))
    if status is not None and int(status.item()) != 0:
        raise RuntimeError("ixb_fa_bwd: an internal pipeline wait gave up; gradients are undefined")
    return dq, dk, dv


# ---- context-parallel attention merge ----------------------------------------------------
def _stat_nstride(t: torch.Tensor, S: int) -> int:
    """Element stride of the N axis of a ``[B, N, S, 8]`` statistics tensor whose last two
    axes are dense and whose B axis is ``N`` times the N stride (a slice along S of a longer
    buffer qualifies)."""
    B, N = t.shape[0], t.shape[1]
    if t.stride(3) != 1 or t.stride(2) != 8 or (B > 1 and t.stride(0) != N * t.stride(1)):
        raise ValueError("statistics must be [B, N, S, 8] with dense trailing axes")
    return t.stride(1) if N > 1 else S * 8


def forward_update(prev_attn_out: torch.Tensor, prev_softmax_max: torch.Tensor,
                   prev_softmax_sum: torch.Tensor, cur_attn_out: torch.Tensor,
                   cur_softmax_max: torch.Tensor, cur_softmax_sum: torch.Tensor):
    """Merge the attention result of one ring step into the running result, (max, sum) form.
    Same name, arguments and return value ``(attn_out, softmax_max, softmax_sum)`` as the
    reference's ``forward_update`` / ``forward_update_triton``
    (``test/npu_indexing/attn_cp_test.py:36-59``,
    ``test/npu_indexing/written/attn_cp_triton_kernel_3d.py:85-140``): attention outputs are
    ``[S, B, H]``, statistics ``[B, N, S, 8]`` fp32."""
    _need_cuda(prev_attn_out, prev_softmax_max, prev_softmax_sum, cur_attn_out, cur_softmax_max, cur_softmax_sum)
    S, B, H = cur_attn_out.shape
    N = cur_softmax_max.shape[1]
    if prev_attn_out.shape != cur_attn_out.shape or prev_attn_out.dtype != cur_attn_out.dtype:
        raise ValueError("prev and cur attention outputs must share shape and dtype")
    if H % N != 0:
        raise ValueError("hidden size must be a multiple of the number of heads")
    for t in (prev_softmax_max, prev_softmax_sum, cur_softmax_max, cur_softmax_sum):
        if t.dtype != torch.float32 or tuple(t.shape) != (B, N, S, 8):
            raise ValueError("statistics must be fp32 [B, N, S, 8]")
    if not (prev_attn_out.is_contiguous() and cur_attn_out.is_contiguous()):
        raise ValueError("attention outputs must be contiguous [S, B, H]")
    pns, cns = _stat_nstride(prev_softmax_max, S), _stat_nstride(cur_softmax_max, S)
    if _stat_nstride(prev_softmax_sum, S) != pns or _stat_nstride(cur_softmax_sum, S) != cns:
        raise ValueError("max and sum of one side must share their layout")
    attn_out = torch.empty_like(cur_attn_out)
    out_max = torch.empty((B, N, S, 8), dtype=torch.float32, device=cur_attn_out.device)
    out_sum = torch.empty_like(out_max)
    rt.check("ixb_cp_forward_update", rt.load().ixb_cp_forward_update(
        rt.DTYPE_CODE[cur_attn_out.dtype], prev_attn_out.data_ptr(), prev_softmax_max.data_ptr(),
        prev_softmax_sum.data_ptr(), cur_attn_out.data_ptr(), cur_softmax_max.data_ptr(),
        cur_softmax_sum.data_ptr(), attn_out.data_ptr(), out_max.data_ptr(), out_sum.data_ptr(),
        S, B, N, H // N, pns, cns, S * 8, rt.raw_stream(cur_attn_out.device)))
    return attn_out, out_max, out_sum


def forward_update_la(prev_attn_out: torch.Tensor, prev_softmax_log_max_sum: torch.Tensor,
                      cur_attn_out: torch.Tensor, cur_softmax_log_max_sum: torch.Tensor) -> None:
    """Log-sum-exp form of the ring merge, in place on ``prev_attn_out`` ``[B, N, S, D]`` fp32
    and ``prev_softmax_log_max_sum`` ``[B, N, S]`` fp32 (the reference's
    ``forward_update_triton`` of ``test/npu_indexing/written/attn_cp_triton_kernel_3d_la.py:58-96``)."""
    _need_cuda(prev_attn_out, prev_softmax_log_max_sum, cur_attn_out, cur_softmax_log_max_sum)
    B, N, S, D = cur_attn_out.shape
    for a in (prev_attn_out, cur_attn_out):
        if a.dtype != torch.float32 or tuple(a.shape) != (B, N, S, D) or a.stride(3) != 1 or a.stride(2) != D \
                or (B > 1 and a.stride(0) != N * a.stride(1)):
            raise ValueError("attention outputs must be fp32 [B, N, S, D] with dense trailing axes")
    for l in (prev_softmax_log_max_sum, cur_softmax_log_max_sum):
        if l.dtype != torch.float32 or tuple(l.shape) != (B, N, S) or l.stride(2) != 1 \
                or (B > 1 and l.stride(0) != N * l.stride(1)):
            raise ValueError("log-sum-exp tensors must be fp32 [B, N, S] with a dense S axis")
    ns = lambda t, dense: t.stride(1) if N > 1 else dense
    rt.check("ixb_cp_forward_update_lse", rt.load().ixb_cp_forward_update_lse(
        prev_attn_out.data_ptr(), prev_softmax_log_max_sum.data_ptr(), cur_attn_out.data_ptr(),
        cur_softmax_log_max_sum.data_ptr(), B, N, S, D, ns(prev_attn_out, S * D),
        ns(prev_softmax_log_max_sum, S), ns(cur_attn_out, S * D), ns(cur_softmax_log_max_sum, S),
        rt.raw_stream(cur_attn_out.device)))


def grad_accumulate(acc: torch.Tensor, cur: torch.Tensor) -> torch.Tensor:
    """``acc.add_(cur.view(acc.shape))`` for dense tensors: the gradient accumulation steps of
    the reference's ring backward (``backward_update``,
    ``test/npu_indexing/written/test_attn_cp.py:267-287``)."""
    _need_cuda(acc, cur)
    if acc.dtype != cur.dtype or acc.numel() != cur.numel() or not (acc.is_contiguous() and cur.is_contiguous()):
        raise ValueError("acc and cur must be dense tensors of one dtype and size")
    rt.check("ixb_cp_accumulate", rt.load().ixb_cp_accumulate(
        rt.DTYPE_CODE[acc.dtype], acc.data_ptr(), cur.data_ptr(), acc.numel(), rt.raw_stream(acc.device)))
    return acc
