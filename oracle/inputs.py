"""Seeded synthetic inputs of the benchmark configurations.  Test infrastructure only.

One CPU ``torch.Generator`` per configuration, tensors drawn in fp32 in the order listed
and then cast, so every consumer (oracle, GPU tests, bench) sees identical bits.  No
public dataset is involved: the reference measures on none.
"""
from __future__ import annotations

import math
from typing import Dict

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def c1(rows: int = 8192, cols: int = 1024, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Fused pointwise + row-sum, fp32: x, w, b ~ N(0,1)."""
    g = _gen(seed)
    return {
        "x": torch.randn(rows, cols, generator=g),
        "w": torch.randn(cols, generator=g),
        "b": torch.randn(cols, generator=g),
    }


def c2(rows: int = 16384, cols: int = 4096, seed: int = 0, dtype=torch.bfloat16):
    """Softmax -> LayerNorm chain: x ~ N(0, sigma=2); g, gamma ~ N(1, 0.1); beta ~ N(0, 0.1).
    (The distribution of g is not given by the benchmark definition; N(1, 0.1) is used.)"""
    g = _gen(seed)
    x = torch.randn(rows, cols, generator=g) * 2.0
    gg = 1.0 + 0.1 * torch.randn(cols, generator=g)
    gamma = 1.0 + 0.1 * torch.randn(cols, generator=g)
    beta = 0.1 * torch.randn(cols, generator=g)
    return {"x": x.to(dtype), "g": gg.to(dtype), "gamma": gamma.to(dtype), "beta": beta.to(dtype)}


def c3a(shape=(64, 128, 256, 64), seed: int = 0, dtype=torch.float16):
    """Permuted / strided reductions: x ~ U(-1, 1), contiguous [a, b, c, d]."""
    g = _gen(seed)
    x = torch.rand(*shape, generator=g) * 2.0 - 1.0
    return {"x": x.to(dtype)}


def c3b(n_rows: int = 1 << 20, dim: int = 128, n_idx: int = 262144, seed: int = 0,
        dtype=torch.float16):
    """index_select: table ~ U(-1, 1) ("1M" rows taken as 2**20), idx ~ U[0, n_rows)."""
    g = _gen(seed)
    table = torch.rand(n_rows, dim, generator=g) * 2.0 - 1.0
    idx = torch.randint(0, n_rows, (n_idx,), generator=g, dtype=torch.int64)
    return {"table": table.to(dtype), "idx": idx}


def c4(B: int = 8, H: int = 32, S: int = 4096, D: int = 128, seed: int = 0, dtype=torch.bfloat16):
    """Fused attention: Q, K, V ~ N(0,1) in [B, H, S, D]; causal; scale 1/sqrt(D)."""
    g = _gen(seed)
    q = torch.randn(B, H, S, D, generator=g)
    k = torch.randn(B, H, S, D, generator=g)
    v = torch.randn(B, H, S, D, generator=g)
    return {"q": q.to(dtype), "k": k.to(dtype), "v": v.to(dtype), "scale": 1.0 / math.sqrt(D)}


def c4_pattern(B: int = 2, S: int = 96, N: int = 3, D: int = 64, seed: int = 4):
    """fp32 [B, S, N, D] inputs for the reference's un-masked search pattern
    (inductor_x/npu_fusion_attention_graph.py:140-147) with inv_scale_factor = sqrt(D)."""
    g = _gen(seed)
    q = torch.randn(B, S, N, D, generator=g)
    k = torch.randn(B, S, N, D, generator=g)
    v = torch.randn(B, S, N, D, generator=g)
    return {"query": q, "key": k, "value": v, "inv_scale_factor": math.sqrt(D)}


def c5_weights(hidden: int = 4096, heads: int = 32, ffn: int = 11008, seed: int = 0,
               dtype=torch.bfloat16):
    """Llama-style decoder layer weights ~ N(0, 0.02) (norm weights are ones)."""
    g = _gen(seed)

    def w(*shape):
        return (0.02 * torch.randn(*shape, generator=g)).to(dtype)

    return {
        "wq": w(hidden, hidden), "wk": w(hidden, hidden), "wv": w(hidden, hidden),
        "wo": w(hidden, hidden), "w_gate": w(ffn, hidden), "w_up": w(ffn, hidden),
        "w_down": w(hidden, ffn),
        "norm1": torch.ones(hidden, dtype=dtype), "norm2": torch.ones(hidden, dtype=dtype),
    }


def c5_input(batch: int = 16, seq: int = 2048, hidden: int = 4096, seed: int = 1,
             dtype=torch.bfloat16):
    g = _gen(seed)
    return torch.randn(batch, seq, hidden, generator=g).to(dtype)


def rope_tables(seq: int, head_dim: int, theta: float = 1e4):
    """cos / sin tables [seq, head_dim] of rotary embeddings (half-split convention)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq, dtype=torch.float32), inv)
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def cp_merge(S: int = 8192, B: int = 1, H: int = 6144, N: int = 48, seed: int = 7, dtype=torch.bfloat16):
    """Inputs of one ring-attention merge step with the shapes of the reference's own
    profile case ((S, B, H, N) = (4096, 1, 6144, 48) over a doubled sequence,
    test/npu_indexing/written/test_attn_cp.py:241-252): attention outputs [S, B, H],
    statistics [B, N, S, 8] with the eight entries of a row equal."""
    g = _gen(seed)
    rep = lambda t: t.unsqueeze(3).repeat(1, 1, 1, 8)
    return {
        "prev_attn_out": torch.randn((S, B, H), generator=g).to(dtype),
        "prev_softmax_max": rep(torch.rand((B, N, S), generator=g)),
        "prev_softmax_sum": rep(torch.rand((B, N, S), generator=g) + 0.5),
        "cur_attn_out": torch.randn((S, B, H), generator=g).to(dtype),
        "cur_softmax_max": rep(torch.rand((B, N, S), generator=g)),
        "cur_softmax_sum": rep(torch.rand((B, N, S), generator=g) + 0.5),
    }
