"""Eager-PyTorch restatement of the benchmark graphs on CPU.  Test infrastructure only.

Each function computes what the reference's compiled graph computes: half inputs are
widened to fp32 on load (``inductor_x/codegen/triton.py:1431-1433``), the whole fused
graph runs in fp32 (``compute=torch.float32``) or fp64 (truth run), and only the final
result is rounded to the storage dtype.  ``eager_*`` variants run the graph exactly as
the reference's tests run their eager side (``test/npu_indexing/reduction_test.py:28-30``).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------- config 1
def affine_gelu_rowsum(x, w, b, compute=torch.float32):
    """sum(gelu(x*w+b), -1) with erf GELU.  Reference lowering: mul
    (``inductor_x/lowering.py:251-268``), extern gelu, sum_ with fp32 accumulation
    (``inductor_x/lowering.py:204-215``)."""
    v = x.to(compute) * w.to(compute) + b.to(compute)
    return F.gelu(v).sum(dim=-1).to(x.dtype)


# ----------------------------------------------------------------------------- config 2
def softmax_layernorm(x, g, gamma, beta, eps=1e-5, compute=torch.float32, round_output=True):
    """layer_norm(softmax(x,-1)*g + x).  Mean and variance in the two-pass form the
    reference lowers var_mean to (``inductor_x/lowering.py:270-325``)."""
    xf = x.to(compute)
    t = torch.softmax(xf, dim=-1) * g.to(compute) + xf
    mean = t.mean(dim=-1, keepdim=True)
    var = ((t - mean) ** 2).mean(dim=-1, keepdim=True)
    y = (t - mean) * torch.rsqrt(var + eps) * gamma.to(compute) + beta.to(compute)
    return y.to(x.dtype) if round_output else y


def eager_softmax_layernorm(x, g, gamma, beta, eps=1e-5):
    """The same graph as a user writes it, each op rounding to the storage dtype."""
    t = torch.softmax(x, dim=-1) * g + x
    return F.layer_norm(t, (x.shape[-1],), gamma, beta, eps)


# ----------------------------------------------------------------------------- config 3
def permuted_amax(x, compute=torch.float32):
    """x[a,b,c,d] viewed as (0,2,1,3) then amax over dim 1 -> [a, b, d]."""
    return x.permute(0, 2, 1, 3).to(compute).amax(dim=1).to(x.dtype)


def permuted_sum(x, compute=torch.float32):
    """x[a,b,c,d] viewed as (0,2,1,3) then sum over dim 3 -> [a, c, b]; fp32 accumulation
    for half inputs (``inductor_x/lowering.py:204-233``)."""
    return x.permute(0, 2, 1, 3).to(compute).sum(dim=3).to(x.dtype)


def index_select_rows(table, idx):
    """Bit-exact gather along dim 0."""
    return table.index_select(0, idx)


# ----------------------------------------------------------------------------- config 4
def attention_pattern(query, key, value, inv_scale_factor, dropout_p=0.0):
    """The reference's search pattern executed eagerly on [B, S, N, D] inputs
    (``inductor_x/npu_fusion_attention_graph.py:140-147``)."""
    q = query.permute(0, 2, 1, 3)
    k = key.permute(0, 2, 1, 3)
    v = value.permute(0, 2, 1, 3)
    return F.dropout(
        torch.matmul(q, k.transpose(-2, -1)).div(inv_scale_factor).softmax(dim=-1), p=dropout_p
    ).matmul(v)


def attention(q, k, v, scale, causal=True, compute=torch.float32):
    """softmax(q k^T * scale [+ causal mask]) v on [B, H, S, D]; one (batch, head) at a
    time so the score matrix stays small.  Returns (out in q.dtype, log-sum-exp fp32)."""
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    out = torch.empty_like(q)
    lse = torch.empty(B, H, Sq, dtype=torch.float32)
    mask = None
    if causal:
        mask = torch.ones(Sq, Sk, dtype=torch.bool).tril(diagonal=Sk - Sq)
    for b in range(B):
        for h in range(H):
            s = (q[b, h].to(compute) @ k[b, h].to(compute).t()) * scale
            if mask is not None:
                s = s.masked_fill(~mask, float("-inf"))
            lse[b, h] = torch.logsumexp(s, dim=-1).float()
            out[b, h] = (torch.softmax(s, dim=-1) @ v[b, h].to(compute)).to(q.dtype)
    return out, lse


def attention_backward(q, k, v, dout, scale, causal=True):
    """(dq, dk, dv) of `attention` by autograd through its fp32 eager form, one (batch, head)
    at a time.  The reference delegates these gradients to the vendor call
    torch_npu.npu_fusion_attention_grad (``inductor_x/npu_fusion_attention_graph.py:38-42``),
    which is not in its tree: this restates the published math, parity unpinned."""
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    dq, dk, dv = torch.empty_like(q, dtype=torch.float32), torch.empty_like(k, dtype=torch.float32), \
        torch.empty_like(v, dtype=torch.float32)
    mask = torch.ones(Sq, Sk, dtype=torch.bool).tril(diagonal=Sk - Sq) if causal else None
    for b in range(B):
        for h in range(H):
            qf, kf, vf = (t[b, h].float().clone().requires_grad_(True) for t in (q, k, v))
            s = (qf @ kf.t()) * scale
            if mask is not None:
                s = s.masked_fill(~mask, float("-inf"))
            (torch.softmax(s, dim=-1) @ vf).backward(dout[b, h].float())
            dq[b, h], dk[b, h], dv[b, h] = qf.grad, kf.grad, vf.grad
    return dq, dk, dv


# ----------------------------------------------------------------------------- config 5
def rmsnorm(x, w, eps=1e-6, compute=torch.float32):
    xf = x.to(compute)
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.to(compute)).to(x.dtype)


def add_rmsnorm(x, res, w, eps=1e-6, compute=torch.float32):
    """h = x + res (rounded to storage dtype), y = rmsnorm(h)."""
    h = (x.to(compute) + res.to(compute)).to(x.dtype)
    return rmsnorm(h, w, eps, compute), h


def rope(x, cos, sin, compute=torch.float32):
    """Rotary embedding, half-split convention, x [B, H, S, D], tables [S, D]."""
    xf = x.to(compute)
    d = x.shape[-1] // 2
    rot = torch.cat([-xf[..., d:], xf[..., :d]], dim=-1)
    return (xf * cos.to(compute) + rot * sin.to(compute)).to(x.dtype)


def swiglu(gate, up, compute=torch.float32):
    return (F.silu(gate.to(compute)) * up.to(compute)).to(gate.dtype)


def llama_layer(x, w, heads=32, eps=1e-6, theta=1e4, compute=torch.float32):
    """Llama-style decoder layer; GEMMs in `compute`, storage rounding between ops as the
    compiled graph would have it at kernel boundaries."""
    from .inputs import rope_tables

    B, S, Hd = x.shape
    D = Hd // heads
    dt = x.dtype

    def mm(a, wt):
        return (a.to(compute) @ wt.to(compute).t()).to(dt)

    h1 = rmsnorm(x, w["norm1"], eps, compute)
    q = mm(h1, w["wq"]).view(B, S, heads, D).transpose(1, 2)
    k = mm(h1, w["wk"]).view(B, S, heads, D).transpose(1, 2)
    v = mm(h1, w["wv"]).view(B, S, heads, D).transpose(1, 2)
    cos, sin = rope_tables(S, D, theta)
    q, k = rope(q, cos, sin, compute), rope(k, cos, sin, compute)
    a, _ = attention(q.contiguous(), k.contiguous(), v.contiguous(), 1.0 / math.sqrt(D), True, compute)
    a = a.transpose(1, 2).reshape(B, S, Hd)
    o = mm(a, w["wo"])
    h2, res = add_rmsnorm(o, x, w["norm2"], eps, compute)
    ff = mm(swiglu(mm(h2, w["w_gate"]), mm(h2, w["w_up"]), compute), w["w_down"])
    return (ff.to(compute) + res.to(compute)).to(dt)


# --------------------------------------------------------------------------- tolerances
def tolerance(dtype):
    """Relative tolerance of the parity bar: 1e-5 for fp32 reductions, 2e-2 for half."""
    return 1e-5 if dtype == torch.float32 else 2e-2


def max_rel_err(actual, expected, floor=None, dim=None):
    """max |a - e| / max(|e|, floor); floor defaults to the RMS of e so that values near
    zero do not dominate (LayerNorm / attention outputs are centred on zero).  With `dim`
    the RMS is taken per slice along that axis: rows of a causal attention output differ
    in scale by orders of magnitude (row i averages i+1 values), so each row is judged
    against its own magnitude."""
    a, e = actual.double(), expected.double()
    if floor is None:
        if dim is None:
            floor = float(e.pow(2).mean().sqrt()) or 1.0
        else:
            floor = e.pow(2).mean(dim, keepdim=True).sqrt().clamp_min(1e-30)
            return float(((a - e).abs() / torch.maximum(e.abs(), floor)).max())
    return float(((a - e).abs() / e.abs().clamp_min(floor)).max())


# ---- context-parallel attention merge (ring step) ----------------------------------------
def cp_forward_update(prev_attn_out, prev_softmax_max, prev_softmax_sum, cur_attn_out, cur_softmax_max,
                      cur_softmax_sum):
    """Eager (max, sum) merge, as the reference states it
    (test/npu_indexing/attn_cp_test.py:24-59): statistics [B, N, S, 8], attention outputs
    [S, B, H]; the scale of an output element comes from entry 0 of its (b, n, s) row."""
    org_dtype = prev_attn_out.dtype
    softmax_max = torch.maximum(prev_softmax_max, cur_softmax_max)
    prev_scaled = prev_softmax_sum * torch.exp(prev_softmax_max - softmax_max)
    cur_scaled = cur_softmax_sum * torch.exp(cur_softmax_max - softmax_max)
    softmax_sum = prev_scaled + cur_scaled

    def to_sbh(x):  # [B, N, S, 8] -> [S, B, N*D]
        b, n, s, _ = x.shape
        d = prev_attn_out.shape[-1] // n
        return x[..., 0].unsqueeze(3).expand(b, n, s, d).permute(2, 0, 1, 3).reshape(s, b, n * d)

    attn = prev_attn_out.float() * to_sbh(prev_scaled / softmax_sum) + \
        cur_attn_out.float() * to_sbh(cur_scaled / softmax_sum)
    return attn.to(org_dtype), softmax_max, softmax_sum


def cp_forward_update_la(prev_attn_out, prev_lse, cur_attn_out, cur_lse):
    """Eager log-sum-exp merge; returns the new (attn_out, lse) instead of updating in place
    (test/npu_indexing/written/attn_cp_triton_kernel_3d_la.py:43-55)."""
    lse = torch.logaddexp(prev_lse.double(), cur_lse.double())
    attn = torch.exp(prev_lse.double() - lse).unsqueeze(-1) * prev_attn_out.double() + \
        torch.exp(cur_lse.double() - lse).unsqueeze(-1) * cur_attn_out.double()
    return attn.float(), lse.float()
