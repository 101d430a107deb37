"""Fused-attention graph pass: SDPA-shaped subgraphs -> the tcgen05 flash-attention kernel.

Surface kept from ``inductor_x/npu_fusion_attention_graph.py``:

* custom ops ``<ns>::b200_fa`` / ``b200_fa_backward`` with the reference's 19-argument /
  27-argument schemas (``:13-18``), a CUDA implementation (``:20-42``) and a Meta
  implementation (``:45-86``);
* the autograd wrapper and public entry ``b200_fusion_attention_graph`` (``:88-132``);
* ``register_fx_pass`` registering the reference's search pattern - permute x3,
  ``matmul . div(inv_scale) . softmax . dropout . matmul`` - in training and inference
  variants into ``joint_graph.patterns`` (``:134-230``).

Additions the benchmark graphs need and the reference lacks (its only pattern has no mask):
a device graph pass that retargets ``aten._scaled_dot_product_*_attention`` nodes - what
``F.scaled_dot_product_attention(..., is_causal=True)`` and the stock causal-mask patterns
become - to the same kernel.

Scale convention: as in the reference, the op's ``scale`` argument carries
``inv_scale_factor`` and the implementation inverts it before calling the kernel
(``:22-29,162``).  ``softmax_max`` / ``softmax_sum`` are returned as ``(logsumexp, 1)``
broadcast to ``[B, N, S, 8]``: an equivalent (max, sum) pair for ``exp(s - max) / sum``.
"""
from __future__ import annotations

import functools
from typing import Optional

import torch
import torch.nn.functional as F
from torch.autograd import Function
from torch.library import Library

TOKEN_MAX = 2147483647
NAMESPACE = "b200_graph"

b200_def = Library(NAMESPACE, "DEF")
b200_def.define(
    "b200_fa(Tensor query, Tensor key, Tensor value, int head_num, str input_layout, Tensor? pse=None, "
    "Tensor? padding_mask=None, Tensor? atten_mask=None, float scale=1., float keep_prob=1., "
    "int pre_tockens=2147483647, int next_tockens=2147483647, int inner_precise=0, int[]? prefix=None, "
    "int[]? actual_seq_qlen=None, int[]? actual_seq_kvlen=None, int sparse_mode=0, "
    "bool gen_mask_parallel=True, bool sync=False) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)")
b200_def.define(
    "b200_fa_backward(Tensor query, Tensor key, Tensor value, Tensor dy, int head_num, str input_layout, *, "
    "Tensor? pse=None, Tensor? padding_mask=None, Tensor? atten_mask=None, Tensor? softmax_max=None, "
    "Tensor? softmax_sum=None, Tensor? softmax_in=None, Tensor? attention_in=None, float scale_value=1., "
    "float keep_prob=1., int pre_tockens=2147483647, int next_tockens=2147483647, int inner_precise=0, "
    "Tensor? seed=None, Tensor? offset=None, Tensor? numels=None, int[]? prefix=None, "
    "int[]? actual_seq_qlen=None, int[]? actual_seq_kvlen=None, int sparse_mode=0, "
    "bool gen_mask_parallel=True, bool sync=False) -> (Tensor, Tensor, Tensor, Tensor)")
# compact form used by the SDPA retargeting pass: (out, logsumexp)
b200_def.define("b200_sdpa(Tensor query, Tensor key, Tensor value, float scale, bool is_causal) -> (Tensor, Tensor)")
b200_def.define("b200_sdpa_backward(Tensor query, Tensor key, Tensor value, Tensor out, Tensor lse, Tensor dout, "
                "float scale, bool is_causal) -> (Tensor, Tensor, Tensor)")

b200_cuda = Library(NAMESPACE, "IMPL", "CUDA")
b200_meta = Library(NAMESPACE, "IMPL", "Meta")

CAUSAL_SPARSE_MODES = (2, 3)  # left-up / right-down aligned causal masks


def _to_bnsd(t: torch.Tensor, layout: str, head_num: int) -> torch.Tensor:
    if layout == "BNSD":
        return t
    if layout == "BSND":
        return t.transpose(1, 2)
    if layout == "BSH":
        b, s, h = t.shape
        return t.view(b, s, head_num, h // head_num).transpose(1, 2)
    if layout == "SBH":
        s, b, h = t.shape
        return t.view(s, b, head_num, h // head_num).permute(1, 2, 0, 3)
    raise ValueError(f"unsupported input_layout {layout!r}")


def _from_bnsd(t: torch.Tensor, layout: str) -> torch.Tensor:
    if layout == "BNSD":
        return t
    if layout == "BSND":
        return t.transpose(1, 2).contiguous()
    b, n, s, d = t.shape
    if layout == "BSH":
        return t.transpose(1, 2).reshape(b, s, n * d)
    return t.permute(2, 0, 1, 3).reshape(s, b, n * d)


def _run_kernel(q, k, v, scale: float, causal: bool):
    from . import ops

    from . import config

    dt = q.dtype
    if dt == torch.float32:
        # the reference traces its pattern in fp32 only (:174); the tensor-core kernel takes
        # 16-bit operands.  Narrowing is the caller's decision, never a silent one: fp16
        # keeps three more mantissa bits than bf16
        if not config.attention_fp32_as_fp16:
            raise TypeError("b200_fa: float32 operands would be narrowed to float16 for the tensor-core "
                            "kernel; set IXB_ATTENTION_FP32_AS_FP16=1 (config.attention_fp32_as_fp16) to allow it")
        q, k, v = q.to(torch.float16), k.to(torch.float16), v.to(torch.float16)
    if q.stride(-1) != 1:
        q = q.contiguous()
    if k.stride(-1) != 1:
        k = k.contiguous()
    if v.stride(-1) != 1:
        v = v.contiguous()
    out, lse = ops.fused_attention(q, k, v, scale, causal=causal, return_lse=True)
    return out.to(dt), lse


def b200_fa_impl(query, key, value, head_num, input_layout, pse=None, padding_mask=None,
                 atten_mask=None, scale=1.0, keep_prob=1.0, pre_tockens=TOKEN_MAX, next_tockens=TOKEN_MAX,
                 inner_precise=0, prefix=None, actual_seq_qlen=None, actual_seq_kvlen=None, sparse_mode=0,
                 gen_mask_parallel=True, sync=False):
    if pse is not None or padding_mask is not None or keep_prob != 1.0:
        raise NotImplementedError("b200_fa: pse, padding_mask and dropout are not supported")
    causal = sparse_mode in CAUSAL_SPARSE_MODES
    if atten_mask is not None and not causal:
        raise NotImplementedError("b200_fa: only causal masks (sparse_mode 2 or 3) are supported")
    q = _to_bnsd(query, input_layout, head_num)
    k = _to_bnsd(key, input_layout, head_num)
    v = _to_bnsd(value, input_layout, head_num)
    if sparse_mode == 2 and q.shape[2] != k.shape[2]:
        raise NotImplementedError("b200_fa: left-up causal needs equal sequence lengths")
    # the op receives inv_scale_factor; the kernel wants the multiplier
    out, lse = _run_kernel(q, k, v, 1.0 / scale, causal)
    b, n, s, _ = out.shape
    smax = lse.unsqueeze(-1).expand(b, n, s, 8).contiguous()
    ssum = torch.ones_like(smax)
    zero = lambda: torch.zeros(1, dtype=torch.int64)
    return (_from_bnsd(out, input_layout), smax, ssum, torch.empty(0, dtype=query.dtype, device=query.device),
            zero(), zero(), zero())


def b200_fa_meta(query, key, value, head_num, input_layout, pse=None, padding_mask=None, atten_mask=None,
                 scale=1.0, keep_prob=1.0, pre_tockens=TOKEN_MAX, next_tockens=TOKEN_MAX, inner_precise=0,
                 prefix=None, actual_seq_qlen=None, actual_seq_kvlen=None, sparse_mode=0,
                 gen_mask_parallel=True, sync=False):
    if input_layout == "BSH":
        b, s1 = query.size(0), query.size(1)
    elif input_layout == "SBH":
        b, s1 = query.size(1), query.size(0)
    elif input_layout == "BSND":
        b, s1 = query.size(0), query.size(1)
    else:
        b, s1 = query.size(0), query.size(2)
    stats = torch.empty([b, head_num, s1, 8], dtype=torch.float32, device="meta")
    return (torch.empty_like(query, device="meta").contiguous(), stats, torch.empty_like(stats),
            torch.empty([0], dtype=query.dtype, device="meta"),
            torch.empty([1], dtype=torch.int64, device="meta"),
            torch.empty([1], dtype=torch.int64, device="meta"),
            torch.empty([1], dtype=torch.int64, device="meta"))


def _run_backward_kernel(q, k, v, out, lse, dout, scale: float, causal: bool):
    """(dq, dk, dv) in the dtype of q from the tcgen05 backward kernels (BNSD views)."""
    from . import config, ops

    dt = q.dtype
    if dt == torch.float32:
        if not config.attention_fp32_as_fp16:
            raise TypeError("b200_fa_backward: float32 operands would be narrowed to float16 for the "
                            "tensor-core kernel; set IXB_ATTENTION_FP32_AS_FP16=1 to allow it")
        q, k, v, out, dout = (t.to(torch.float16) for t in (q, k, v, out, dout))
    fix = lambda t: t if t.stride(-1) == 1 and all(st % 8 == 0 for st in t.stride()[:3]) else t.contiguous()
    dq, dk, dv = ops.fused_attention_backward(fix(q), fix(k), fix(v), fix(out), lse, fix(dout), scale,
                                              causal=causal)
    return dq.to(dt), dk.to(dt), dv.to(dt)


def b200_fa_backward_impl(query, key, value, dy, head_num, input_layout, *, pse=None, padding_mask=None,
                          atten_mask=None, softmax_max=None, softmax_sum=None, softmax_in=None,
                          attention_in=None, scale_value=1.0, keep_prob=1.0, pre_tockens=TOKEN_MAX,
                          next_tockens=TOKEN_MAX, inner_precise=0, seed=None, offset=None, numels=None,
                          prefix=None, actual_seq_qlen=None, actual_seq_kvlen=None, sparse_mode=0,
                          gen_mask_parallel=True, sync=False):
    """Gradients of the fused attention from the statistics the forward saved
    (``npu_fusion_attention_graph.py:38-42``).  The log-sum-exp is rebuilt from the
    ``(softmax_max, softmax_sum)`` pair, the probabilities are recomputed tile by tile inside
    the tcgen05 kernels behind ``ixb_fa_bwd``; as in the forward op, ``scale_value`` carries
    ``inv_scale_factor``."""
    if pse is not None or padding_mask is not None or keep_prob != 1.0:
        raise NotImplementedError("b200_fa_backward: pse, padding_mask and dropout are not supported")
    if softmax_max is None or softmax_sum is None or attention_in is None:
        raise ValueError("b200_fa_backward needs softmax_max, softmax_sum and attention_in from the forward")
    causal = sparse_mode in CAUSAL_SPARSE_MODES
    if atten_mask is not None and not causal:
        raise NotImplementedError("b200_fa_backward: only causal masks (sparse_mode 2 or 3) are supported")
    q = _to_bnsd(query, input_layout, head_num)
    k = _to_bnsd(key, input_layout, head_num)
    v = _to_bnsd(value, input_layout, head_num)
    o = _to_bnsd(attention_in, input_layout, head_num)
    do = _to_bnsd(dy, input_layout, head_num)
    if sparse_mode == 2 and q.shape[2] != k.shape[2]:
        raise NotImplementedError("b200_fa_backward: left-up causal needs equal sequence lengths")
    lse = softmax_max[..., 0] + torch.log(softmax_sum[..., 0])           # [B, N, Sq]
    dq, dk, dv = _run_backward_kernel(q, k, v, o, lse, do, 1.0 / scale_value, causal)
    return (_from_bnsd(dq, input_layout), _from_bnsd(dk, input_layout), _from_bnsd(dv, input_layout), None)


def b200_fa_backward_meta(query, key, value, dy, head_num, input_layout, **kwargs):
    pse = kwargs.get("pse")
    return (torch.empty_like(query, device="meta"), torch.empty_like(key, device="meta"),
            torch.empty_like(value, device="meta"),
            torch.empty([0], dtype=query.dtype, device="meta") if pse is not None else None)


def b200_sdpa_impl(query, key, value, scale, is_causal):
    return _run_kernel(query, key, value, scale, is_causal)


def b200_sdpa_meta(query, key, value, scale, is_causal):
    b, n, s, d = query.shape
    return (torch.empty((b, n, s, d), dtype=query.dtype, device="meta"),
            torch.empty((b, n, s), dtype=torch.float32, device="meta"))


b200_cuda.impl("b200_fa", b200_fa_impl)
b200_meta.impl("b200_fa", b200_fa_meta)
b200_cuda.impl("b200_fa_backward", b200_fa_backward_impl)
b200_meta.impl("b200_fa_backward", b200_fa_backward_meta)
def b200_sdpa_backward_impl(query, key, value, out, lse, dout, scale, is_causal):
    return _run_backward_kernel(query, key, value, out, lse, dout, scale, is_causal)


def b200_sdpa_backward_meta(query, key, value, out, lse, dout, scale, is_causal):
    new = lambda t: torch.empty(t.shape, dtype=t.dtype, device="meta")
    return new(query), new(key), new(value)


b200_cuda.impl("b200_sdpa", b200_sdpa_impl)
b200_meta.impl("b200_sdpa", b200_sdpa_meta)
b200_cuda.impl("b200_sdpa_backward", b200_sdpa_backward_impl)
b200_meta.impl("b200_sdpa_backward", b200_sdpa_backward_meta)


def _sdpa_setup_context(ctx, inputs, output):
    query, key, value, scale, is_causal = inputs
    out, lse = output
    ctx.save_for_backward(query, key, value, out, lse)
    ctx.scale, ctx.is_causal = scale, is_causal


def _sdpa_backward(ctx, d_out, d_lse):
    query, key, value, out, lse = ctx.saved_tensors
    dq, dk, dv = torch.ops.b200_graph.b200_sdpa_backward(query, key, value, out, lse, d_out, ctx.scale,
                                                         ctx.is_causal)
    return dq, dk, dv, None, None


# gradients of the compact op (the log-sum-exp output is not differentiated through)
torch.library.register_autograd("b200_graph::b200_sdpa", _sdpa_backward, setup_context=_sdpa_setup_context,
                                lib=b200_def)


class B200GraphAttentionFunction(Function):
    """Autograd wrapper (``NpuGraphAttentionFunction``, ``:88-123``): forward on the tcgen05
    kernel, backward through ``b200_fa_backward`` (the tcgen05 backward kernels)."""

    @staticmethod
    def forward(ctx, query, key, value, head_num, input_layout, pse=None, padding_mask=None,
                atten_mask=None, scale=1.0, keep_prob=1.0, pre_tockens=TOKEN_MAX, next_tockens=TOKEN_MAX,
                inner_precise=0, prefix=None, actual_seq_qlen=None, actual_seq_kvlen=None, sparse_mode=0,
                gen_mask_parallel=True, sync=False):
        res = torch.ops.b200_graph.b200_fa(
            query, key, value, head_num, input_layout, pse=pse, padding_mask=padding_mask,
            atten_mask=atten_mask, scale=scale, keep_prob=keep_prob, pre_tockens=pre_tockens,
            next_tockens=next_tockens, inner_precise=inner_precise, prefix=prefix,
            actual_seq_qlen=actual_seq_qlen, actual_seq_kvlen=actual_seq_kvlen, sparse_mode=sparse_mode,
            gen_mask_parallel=gen_mask_parallel, sync=sync)
        ctx.save_for_backward(query, key, value, res[1], res[2], res[0])
        ctx.head_num, ctx.input_layout, ctx.scale = head_num, input_layout, scale
        ctx.sparse_mode = sparse_mode
        return res

    @staticmethod
    def backward(ctx, *grads):
        query, key, value, smax, ssum, out = ctx.saved_tensors
        dq, dk, dv, _ = torch.ops.b200_graph.b200_fa_backward(
            query, key, value, grads[0], ctx.head_num, ctx.input_layout, softmax_max=smax,
            softmax_sum=ssum, attention_in=out, scale_value=ctx.scale, sparse_mode=ctx.sparse_mode)
        return (dq, dk, dv) + (None,) * 16


def b200_fusion_attention_graph(query, key, value, head_num, input_layout, pse=None, padding_mask=None,
                                atten_mask=None, scale=1.0, keep_prob=1.0, pre_tockens=TOKEN_MAX,
                                next_tockens=TOKEN_MAX, inner_precise=0, prefix=None, actual_seq_qlen=None,
                                actual_seq_kvlen=None, sparse_mode=0, gen_mask_parallel=True, sync=False):
    """Public entry (the reference installs it as ``torch_npu.npu_fusion_attention_graph``)."""
    if torch.is_grad_enabled() and any(t.requires_grad for t in (query, key, value)):
        return B200GraphAttentionFunction.apply(
            query, key, value, head_num, input_layout, pse, padding_mask, atten_mask, scale, keep_prob,
            pre_tockens, next_tockens, inner_precise, prefix, actual_seq_qlen, actual_seq_kvlen,
            sparse_mode, gen_mask_parallel, sync)
    return torch.ops.b200_graph.b200_fa(
        query, key, value, head_num, input_layout, pse=pse, padding_mask=padding_mask, atten_mask=atten_mask,
        scale=scale, keep_prob=keep_prob, pre_tockens=pre_tockens, next_tockens=next_tockens,
        inner_precise=inner_precise, prefix=prefix, actual_seq_qlen=actual_seq_qlen,
        actual_seq_kvlen=actual_seq_kvlen, sparse_mode=sparse_mode, gen_mask_parallel=gen_mask_parallel,
        sync=sync)


# ---------------------------------------------------------------------------------------
# FX pattern: the reference's search / replace pair, registered the reference's way
# ---------------------------------------------------------------------------------------
def _b200_fusion_attention_graph_pattern_1(query, key, value, inv_scale_factor, dropout_p):
    q = query.permute(0, 2, 1, 3)
    k = key.permute(0, 2, 1, 3)
    v = value.permute(0, 2, 1, 3)
    return torch.nn.functional.dropout(
        torch.matmul(q, k.transpose(-2, -1)).div(inv_scale_factor).softmax(dim=-1),
        p=dropout_p,
    ).matmul(v)


def _b200_fusion_attention_graph_replacement_1(query, key, value, inv_scale_factor, dropout_p):
    from torch._dynamo.utils import counters

    counters["inductor"]["fuse_attention"] += 1
    head_num = query.size(2)
    return b200_fusion_attention_graph(
        query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), head_num, "BNSD", None,
        atten_mask=None, scale=inv_scale_factor, keep_prob=1.0 - dropout_p)[0]


# The benchmark configuration writes causal attention out literally:
#   matmul(q, k^T) -> * scale (or / inv_scale) -> masked_fill(~keep, -inf) -> softmax -> matmul(v)
# with `keep` a lower-triangular boolean matrix built in the graph (torch.ones(S, S).tril()).
# The reference's pattern file has no masked form (its pattern 1 above is un-masked); these
# two search functions extend the same registration to it.  `keep` is a pattern input; the
# extra check then walks the matched node's producers and accepts the rewrite only if they
# provably form j <= i (what tril decomposes to), so an arbitrary mask is never dropped.
def _masked(s, keep):
    # what masked_fill(~keep, -inf) has become by the time the joint-graph patterns run: a
    # where() against a 0-d full(-inf) (Inductor folds the scalar_tensor of the decomposition)
    return torch.where(~keep, torch.full((), float("-inf"), dtype=s.dtype, device=s.device), s)


def _b200_causal_attention_pattern_mul(query, key, value, keep, scale):
    s = _masked(torch.matmul(query, key.transpose(-2, -1)) * scale, keep)
    return torch.matmul(torch.softmax(s, dim=-1), value)


def _b200_causal_attention_pattern_div(query, key, value, keep, inv_scale):
    s = _masked(torch.matmul(query, key.transpose(-2, -1)) / inv_scale, keep)
    return torch.matmul(torch.softmax(s, dim=-1), value)


def _b200_causal_attention_replacement_mul(query, key, value, keep, scale):
    from torch._dynamo.utils import counters

    counters["inductor"]["fuse_attention"] += 1
    # forward-only graph: the compact op (result and log-sum-exp, no [B, N, S, 8] statistics to
    # materialise); causal with equal lengths, which the extra check established
    return torch.ops.b200_graph.b200_sdpa(query, key, value, scale, True)[0]


def _b200_causal_attention_replacement_div(query, key, value, keep, inv_scale):
    from torch._dynamo.utils import counters

    counters["inductor"]["fuse_attention"] += 1
    return torch.ops.b200_graph.b200_sdpa(query, key, value, 1.0 / inv_scale, True)[0]


def _is_all_true(node) -> bool:
    if not isinstance(node, torch.fx.Node) or node.op != "call_function":
        return False
    if node.target in (aten.full.default,) and len(node.args) >= 2:
        return node.args[1] is True or node.args[1] == 1
    if node.target in (aten.ones.default, aten.ones_like.default):
        return True
    return False


def _iota_axis(node):
    """-1 if ``node`` is arange(n) laid along the last axis ([1, n] / [n]), -2 if along the
    second-to-last ([n, 1]); None otherwise."""
    if not isinstance(node, torch.fx.Node) or node.op != "call_function":
        return None
    if node.target is aten.unsqueeze.default:
        src, dim = node.args
        if isinstance(src, torch.fx.Node) and src.op == "call_function" and src.target is torch.ops.prims.iota.default:
            kw = src.kwargs
            if kw.get("start", 0) == 0 and kw.get("step", 1) == 1:
                return {-2: -1, 0: -1, -1: -2, 1: -2}.get(dim)
    return None


def _is_lower_triangular(node, depth: int = 0) -> bool:
    """True when ``node`` provably computes keep[i, j] = (j <= i): the decomposition of
    ``ones(S, S).tril()`` (``le(sub(iota_j, iota_i), 0)``, possibly and-ed with all-true), its
    mirrored spellings, or an undecomposed ``tril`` of an all-true matrix."""
    if depth > 6 or not isinstance(node, torch.fx.Node) or node.op != "call_function":
        return False
    t, a = node.target, node.args
    if t is aten.logical_and.default or t is aten.bitwise_and.Tensor:
        return (_is_all_true(a[0]) and _is_lower_triangular(a[1], depth + 1)) or \
               (_is_all_true(a[1]) and _is_lower_triangular(a[0], depth + 1))
    if t is aten.tril.default:
        return _is_all_true(a[0]) and (len(a) < 2 or a[1] == 0)
    if t in (aten.le.Scalar, aten.ge.Scalar) and a[1] == 0 and isinstance(a[0], torch.fx.Node) and \
            a[0].target is aten.sub.Tensor:
        lhs, rhs = _iota_axis(a[0].args[0]), _iota_axis(a[0].args[1])
        # le: (j - i) <= 0; ge: (i - j) >= 0
        return (lhs, rhs) == ((-1, -2) if t is aten.le.Scalar else (-2, -1))
    if t in (aten.le.Tensor, aten.ge.Tensor):
        lhs, rhs = _iota_axis(a[0]), _iota_axis(a[1])
        return (lhs, rhs) == ((-1, -2) if t is aten.le.Tensor else (-2, -1))
    return False


def _causal_extra_check(match) -> bool:
    if not _pattern_extra_check(match):
        return False
    q, k, v, keep = (match.kwargs.get(n) for n in ("query", "key", "value", "keep"))
    metas = [getattr(n, "meta", {}).get("val") if n is not None else None for n in (q, k, v, keep)]
    if any(m is None for m in metas):
        return False
    qm, km, vm, mm = metas
    if km.dim() != 4 or vm.dim() != 4 or km.shape != vm.shape or km.shape[:2] != qm.shape[:2] or km.shape[-1] != 128:
        return False
    # top-left and bottom-right causal masks coincide only for equal lengths
    if qm.shape[2] != km.shape[2] or tuple(mm.shape[-2:]) != (qm.shape[2], km.shape[2]) or mm.dtype != torch.bool:
        return False
    if any(int(d) != 1 for d in mm.shape[:-2]):
        return False
    return _is_lower_triangular(keep)


def _pattern_extra_check(match) -> bool:
    """Only shapes the kernel instantiates: head dim 128."""
    from . import config

    q = match.kwargs.get("query")
    meta = getattr(q, "meta", {}).get("val") if q is not None else None
    if meta is None or meta.dim() != 4 or meta.shape[-1] != 128:
        return False
    if meta.dtype == torch.float32:
        return config.attention_fp32_as_fp16      # never narrowed without the caller's consent
    return meta.dtype in (torch.float16, torch.bfloat16)


def _joint_fwd_bwd_folded(fn, args):
    """``joint_fwd_bwd`` with the 0-d ``scalar_tensor`` nodes of the trace (the zero that the
    gradient of ``where`` fills in) rewritten to ``full([], value)``: Inductor's constant
    folding has done that to the joint graph by the time the patterns are matched."""
    from torch._inductor.pattern_matcher import joint_fwd_bwd

    gm = joint_fwd_bwd(fn, args)
    for node in list(gm.graph.nodes):
        if node.op == "call_function" and node.target is aten.scalar_tensor.default:
            with gm.graph.inserting_before(node):
                full = gm.graph.call_function(
                    aten.full.default, ([], node.args[0]),
                    {"dtype": node.kwargs.get("dtype"), "device": node.kwargs.get("device"), "pin_memory": False})
            full.meta.update(node.meta)
            node.replace_all_uses_with(full)
            gm.graph.erase_node(node)
    gm.graph.lint()
    gm.recompile()
    return gm


def _get_sfdp_patterns():
    from torch._inductor.fx_passes.fuse_attention import partialize_and_update_signature
    from torch._inductor.fx_passes.joint_graph import patterns
    from torch._inductor.pattern_matcher import fwd_only, joint_fwd_bwd

    device = "cuda" if torch.cuda.is_available() else "cpu"
    g_inp = functools.partial(torch.empty, (2, 4, 8, 16), device=device, requires_grad=True)
    c_inp = functools.partial(torch.tensor, 2.0, device=device)
    workaround = {"dropout_p": 0.113377}
    # the reference traces float32 only; half types trace differently (casts around the
    # softmax) and are what the kernel takes, so the pattern is registered for them as well
    for dtype in [torch.float, torch.bfloat16, torch.float16]:
        g = functools.partial(g_inp, dtype=dtype)
        c = functools.partial(c_inp, dtype=dtype)
        pattern, replacement = _b200_fusion_attention_graph_pattern_1, _b200_fusion_attention_graph_replacement_1
        args = [g(), g(), g(), c()]
        name = f"{pattern.__name__}_{dtype}"
        # the inference variant drops dropout, exactly as the reference partialises it
        # (:206-216).  The reference's training variant keeps dropout (:196-204), which these
        # kernels do not have (keep_prob != 1 raises); the training variant registered here is
        # the dropout-free form, gradients through b200_fa_backward
        pattern_i = partialize_and_update_signature(pattern, dropout_p=0.0)
        replacement_i = partialize_and_update_signature(replacement, dropout_p=0.0)
        yield name + "_training", {
            "search_fn": pattern_i, "replace_fn": replacement_i, "example_inputs": args,
            "trace_fn": joint_fwd_bwd, "pass_dicts": patterns, "scalar_workaround": {},
            "extra_check": _pattern_extra_check,
        }
        yield name + "_inference", {
            "search_fn": pattern_i, "replace_fn": replacement_i, "example_inputs": args,
            "trace_fn": fwd_only, "pass_dicts": patterns, "scalar_workaround": {},
            "extra_check": _pattern_extra_check,
        }
    # the masked (causal) form, in the dtypes the kernel takes plus float32 (matched only with
    # the fp16 opt-in): half types trace differently (casts around the softmax)
    for dtype in [torch.bfloat16, torch.float16, torch.float]:
        b_inp = functools.partial(torch.empty, (2, 4, 8, 128), device=device, dtype=dtype)
        t_inp = functools.partial(b_inp, requires_grad=True)
        keep = functools.partial(torch.ones, (8, 8), device=device, dtype=torch.bool)
        c = functools.partial(c_inp, dtype=dtype)      # same dtype: no cast node around the scalar
        for pattern, replacement in ((_b200_causal_attention_pattern_mul, _b200_causal_attention_replacement_mul),
                                     (_b200_causal_attention_pattern_div, _b200_causal_attention_replacement_div)):
            # training: forward and backward of the pattern are matched in the joint graph and
            # replaced by b200_sdpa and its registered gradient (b200_sdpa_backward)
            yield f"{pattern.__name__}_{dtype}_training", {
                "search_fn": pattern, "replace_fn": replacement,
                "example_inputs": [t_inp(), t_inp(), t_inp(), keep(), c()],
                "trace_fn": _joint_fwd_bwd_folded, "pass_dicts": patterns, "scalar_workaround": {},
                "extra_check": _causal_extra_check,
            }
            yield f"{pattern.__name__}_{dtype}_inference", {
                "search_fn": pattern, "replace_fn": replacement,
                "example_inputs": [b_inp(), b_inp(), b_inp(), keep(), c()],
                "trace_fn": fwd_only, "pass_dicts": patterns, "scalar_workaround": {},
                "extra_check": _causal_extra_check,
            }


_fx_pass_registered = False


def register_fx_pass():
    """Register the search pattern into ``joint_graph.patterns`` (``:196-230``)."""
    global _fx_pass_registered
    if _fx_pass_registered:
        return
    from torch._inductor.pattern_matcher import register_replacement

    for _key, kwargs in _get_sfdp_patterns():
        register_replacement(**kwargs)
    _fx_pass_registered = True


# ---------------------------------------------------------------------------------------
# Device graph pass: aten SDPA kernels -> b200_sdpa
# ---------------------------------------------------------------------------------------
from torch._inductor.custom_graph_pass import CustomGraphModulePass, get_hash_for_files  # noqa: E402

aten = torch.ops.aten


class B200AttentionPass(CustomGraphModulePass):
    """Rewrites ``aten._scaled_dot_product_{flash,efficient,cudnn}_attention`` nodes whose
    only used output is the attention result (optionally the log-sum-exp) into
    ``b200_graph.b200_sdpa`` when the kernel supports the case: fp16 / bf16, head dim 128,
    no dropout, no additive bias, causal or no mask."""

    def __call__(self, gm: torch.fx.GraphModule) -> None:
        changed = False
        for node in list(gm.graph.nodes):
            if node.op != "call_function":
                continue
            spec = self._match(node)
            if spec is None:
                continue
            q, k, v, scale, causal = spec
            with gm.graph.inserting_before(node):
                new = gm.graph.call_function(torch.ops.b200_graph.b200_sdpa.default, (q, k, v, scale, causal))
            import operator

            ok = True
            for user in list(node.users):
                if user.op == "call_function" and user.target is operator.getitem and user.args[1] in (0, 1):
                    continue
                if len(user.users) == 0:
                    continue
                ok = False
            if not ok:
                gm.graph.erase_node(new)
                continue
            qv = q.meta.get("val")
            new.meta["val"] = (torch.empty_like(qv), qv.new_empty(qv.shape[:3], dtype=torch.float32))
            for user in list(node.users):
                if user.target is operator.getitem and user.args[1] in (0, 1):
                    with gm.graph.inserting_before(user):
                        item = gm.graph.call_function(operator.getitem, (new, user.args[1]))
                    item.meta.update(user.meta)
                    user.replace_all_uses_with(item)
                gm.graph.erase_node(user)
            gm.graph.erase_node(node)
            changed = True
        if changed:
            gm.graph.lint()
            gm.recompile()

    @staticmethod
    def _match(node):
        t = node.target
        flash = getattr(aten._scaled_dot_product_flash_attention, "default", None)
        eff = getattr(aten._scaled_dot_product_efficient_attention, "default", None)
        cudnn = getattr(getattr(aten, "_scaled_dot_product_cudnn_attention", None), "default", None)
        kw = dict(node.kwargs)
        if t is flash:
            q, k, v = node.args[:3]
            dropout = node.args[3] if len(node.args) > 3 else kw.get("dropout_p", 0.0)
            causal = node.args[4] if len(node.args) > 4 else kw.get("is_causal", False)
            bias = None
        elif t is eff or (cudnn is not None and t is cudnn):
            q, k, v = node.args[:3]
            bias = node.args[3] if len(node.args) > 3 else kw.get("attn_bias")
            dropout = node.args[5] if len(node.args) > 5 else kw.get("dropout_p", 0.0)
            causal = node.args[6] if len(node.args) > 6 else kw.get("is_causal", False)
        else:
            return None
        if bias is not None or dropout not in (0, 0.0):
            return None
        qv = q.meta.get("val") if hasattr(q, "meta") else None
        kv = k.meta.get("val") if hasattr(k, "meta") else None
        vv = v.meta.get("val") if hasattr(v, "meta") else None
        if qv is None or kv is None or vv is None or qv.dim() != 4 or qv.shape[-1] != 128:
            return None
        if qv.dtype not in (torch.float16, torch.bfloat16) or qv.device.type != "cuda":
            return None
        # the kernel handles equal head counts, head dim 128 on all three operands, one
        # dtype and ordinary (positive-stride) layouts; anything else stays with the aten kernel
        for t in (kv, vv):
            if t.dim() != 4 or t.shape[0] != qv.shape[0] or t.shape[1] != qv.shape[1] or t.shape[-1] != 128:
                return None
            if t.dtype != qv.dtype or t.device != qv.device:
                return None
        if kv.shape[2] != vv.shape[2]:
            return None
        if any(int(st) <= 0 for t in (qv, kv, vv) for st, n in zip(t.stride(), t.shape) if n > 1):
            return None
        # is_causal in torch masks from the top-left corner (key j visible iff j <= i); the
        # kernel's causal mode is aligned to the bottom-right corner (j <= i + Sk - Sq).  The two
        # agree only for equal lengths, so a causal node with Sk != Sq is left alone.
        if causal and kv.shape[2] != qv.shape[2]:
            return None
        scale = kw.get("scale")
        if scale is None:
            scale = 1.0 / (qv.shape[-1] ** 0.5)
        return q, k, v, float(scale), bool(causal)

    def uuid(self):
        # Part of Inductor's FX-graph cache key.  Everything that changes the text this backend
        # generates for a given graph has to be in it, or a cached wrapper from an earlier
        # setting would be served: the code generator's sources, the template headers and the
        # configuration flags.
        import glob
        import hashlib
        import os

        from . import config
        from .codegen import jit

        here = os.path.dirname(os.path.abspath(__file__))
        files = tuple(sorted(glob.glob(os.path.join(here, "*.py")) + glob.glob(os.path.join(here, "codegen", "*.py"))))
        flags = (config.merged_welford, config.merged_online_softmax, config.debug_bounds, config.fp64_as_fp32,
                 config.attention_fp32_as_fp16)
        h = hashlib.sha256(get_hash_for_files(files))
        h.update(jit._template_digest())
        h.update(repr(flags).encode())
        return h.digest()
