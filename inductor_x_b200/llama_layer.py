"""The Llama-style decoder layer of benchmark configuration 5, written as the plain PyTorch
graph a user would hand to ``torch.compile``: RMSNorm, QKV projections, rotary embedding,
causal attention, output projection, residual, RMSNorm, SwiGLU feed-forward, residual.
It exists so that tests and the benchmark compile the same graph; it is not a model zoo."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    rot = torch.cat([-x[..., d:], x[..., :d]], dim=-1)
    return (x.float() * cos + rot.float() * sin).to(x.dtype)


def decoder_layer(x, w, cos, sin, heads: int = 32, eps: float = 1e-6):
    """x [B, S, hidden]; w: dict of weights as produced by the benchmark's input generator;
    cos / sin [S, head_dim] fp32 tables."""
    B, S, Hd = x.shape
    D = Hd // heads
    h1 = rms_norm(x, w["norm1"], eps)
    q = F.linear(h1, w["wq"]).view(B, S, heads, D).transpose(1, 2)
    k = F.linear(h1, w["wk"]).view(B, S, heads, D).transpose(1, 2)
    v = F.linear(h1, w["wv"]).view(B, S, heads, D).transpose(1, 2)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    a = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=1.0 / math.sqrt(D))
    a = a.transpose(1, 2).reshape(B, S, Hd)
    h = x + F.linear(a, w["wo"])
    h2 = rms_norm(h, w["norm2"], eps)
    ff = F.linear(F.silu(F.linear(h2, w["w_gate"])) * F.linear(h2, w["w_up"]), w["w_down"])
    return h + ff
