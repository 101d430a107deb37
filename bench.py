#!/usr/bin/env python
"""Benchmark of the inductor_x_b200 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line.  The headline workload (default) is the softmax -> LayerNorm chain on
x[16384, 4096] bf16 run the way a user runs it: ``torch.compile`` with this package's
Inductor backend, every fused group a generated instantiation of the CUDA templates
(``--prebuilt`` times the hand-instantiated entry point of the kernel library instead).  One
"step" is one pass of the graph over that batch.  `value` is algorithmic HBM GB/s with inputs
resident in HBM; `e2e` is the same metric with host buffers (pinned H2D of the inputs and D2H
of the result inside the timed region).  The other benchmark configurations (fp32 GELU row
sum, the permuted reductions, the row gather, fused attention, the decoder layer) are timed
after the headline and reported under `configs`, each with its own roofline.

With N > 1 (launched by torch.distributed.run) every rank runs the same per-GPU batch of the
headline (rows sharded, weak scaling, no data-path collective) and the time is the max over
ranks; `configs` then holds the sharded runs of a FIXED global batch (strong scaling) and the
all-gather of the sharded output.

`--impl reference` times the reference's ground truth for this graph - eager PyTorch on the
host cores - on a bounded sample of the same workload (the reference itself needs an Ascend
NPU stack and cannot execute here).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


# --------------------------------------------------------------------------- clocks
class ClockSampler(threading.Thread):
    """Polls NVML (read-only) for SM clock and throttle reasons while the bench runs."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.stop_flag = threading.Event()
        self.max_mhz = None
        self.ok = False

    def run(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            self.ok = True
            while not self.stop_flag.is_set():
                mhz = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                try:
                    reasons = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    reasons = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.samples.append((time.perf_counter(), mhz, reasons))
                time.sleep(0.002)
        except Exception:
            self.ok = False

    def summary(self, t0: float, t1: float):
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        inside = [(m, r) for (t, m, r) in self.samples if t0 <= t <= t1] or \
                 [(m, r) for (_, m, r) in self.samples[-3:]]
        mhz = sorted(m for m, _ in inside)
        bits = 0
        for _, r in inside:
            bits |= r
        names = [n for b, n in self.REASONS.items() if bits & b]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": self.max_mhz,
                "reasons": names, "samples": len(inside)}


# ------------------------------------------------------------------------ workloads
class Workload:
    """One benchmark configuration.  ``graph()`` is the PyTorch function a user compiles;
    ``prebuilt(*tensors)`` is the same computation through the kernel library's tensor-level
    wrapper.  ``bind(path)`` picks which of the two ``op`` runs; both the device-resident
    timing and the end-to-end timing call ``op``."""

    metric = "fused-kernel HBM GB/s"
    unit = "GB/s"
    bound = "hbm"
    path = "compiled"
    n_out_sets = 3          # outputs of the last steps stay alive, so the allocator rotates blocks
    shard_axis = "rows"

    def bind(self, path: str):
        self.path = path
        self.outs = [None] * self.n_out_sets
        if path == "compiled":
            import inductor_x_b200  # noqa: F401  (registers the backend for "cuda")

            # static shapes: a new extent (the row chunks of the end-to-end pipeline) compiles its own module
            self.compiled = torch.compile(self.graph(), dynamic=False)
        return self

    def op(self, *tensors):
        return self.compiled(*tensors) if self.path == "compiled" else self.prebuilt(*tensors)

    def step(self, i):
        self.outs[i % self.n_out_sets] = self.op(*self.args(i))

    def work(self):
        """Algorithmic work of one step in the metric's unit x 1e9 (bytes, or flops / 1e3)."""
        return self.flops() / 1e3 if self.bound == "tensor" else self.algorithmic_bytes()

    def sets(self):
        return len(getattr(self, "xs", [0]))


class SoftmaxLayerNorm(Workload):
    """configs[1]: y = layer_norm(softmax(x,-1)*g + x) on x[16384,4096] bf16."""

    name = "softmax_layernorm_bf16_16384x4096"
    dtype = "bf16"
    rows, cols = 16384, 4096

    def algorithmic_bytes(self):
        return 2 * self.rows * self.cols * 2 + 3 * self.cols * 2  # 268,460,032

    def load_host(self, seed):
        from oracle import inputs  # input generator only (seeded synthetic data)

        self.host = inputs.c2(self.rows, self.cols, seed=seed)
        return self.host

    def setup(self, device, seed, n_sets=4):
        d = self.load_host(seed)
        self.params = [d[k].to(device) for k in ("g", "gamma", "beta")]
        x = d["x"].to(device)
        # distinct buffers per step: a step streams 268 MB (> 126 MB L2) and the next step
        # touches different addresses, so nothing is served from cache
        self.xs = [x] + [x.clone() for _ in range(n_sets - 1)]

    def args(self, i):
        return (self.xs[i % len(self.xs)], *self.params)

    def graph(self):
        import torch.nn.functional as F

        cols = self.cols
        return lambda x, g, ga, be: F.layer_norm(torch.softmax(x, -1) * g + x, (cols,), ga, be, 1e-5)

    def prebuilt(self, x, g, ga, be):
        from inductor_x_b200 import ops

        return ops.softmax_layernorm(x, g, ga, be, 1e-5)

    def op_into(self, out, x):
        """The same graph writing its result into ``out`` (a slot of a larger buffer): the store
        of the kernel goes there directly, no staging copy."""
        if self.path != "compiled":
            from inductor_x_b200 import ops

            return ops.softmax_layernorm(x, *self.params, 1e-5, out=out)
        if not hasattr(self, "compiled_into"):
            fn = self.graph()
            self.compiled_into = torch.compile(lambda x, g, ga, be, out: out.copy_(fn(x, g, ga, be)), dynamic=False)
        return self.compiled_into(x, *self.params, out)

    e2e_chunks = 8     # fewer, larger chunks when several ranks share the host's copy engines

    def e2e_setup(self, device, chunks=None):
        from inductor_x_b200.host_io import HostRowPipeline

        chunks = chunks or self.e2e_chunks
        self.h_x = self.host["x"].pin_memory()
        self.h_y = torch.empty_like(self.h_x).pin_memory()
        self.pipe = HostRowPipeline(device, self.h_x.shape, self.h_x.dtype, self.h_x.shape,
                                    self.h_x.dtype, chunks=chunks)

    def e2e_step(self):
        # upload / compute / download overlapped chunk by chunk (PCIe in both directions)
        self.pipe.run(self.h_x, lambda xc, out: out.copy_(self.op(xc, *self.params)), self.h_y)
        return self.h_x.numel() * 2, self.h_y.numel() * 2

    def cpu_sample(self, rows=1024):
        from oracle import graphs

        d = self.host
        x = d["x"][:rows].contiguous()
        fn = lambda: graphs.eager_softmax_layernorm(x, d["g"], d["gamma"], d["beta"], 1e-5)
        nbytes = 2 * rows * self.cols * 2 + 3 * self.cols * 2
        return fn, nbytes, f"{rows} of {self.rows} rows, eager PyTorch ops"


class AffineGeluRowSum(Workload):
    """configs[0]: out = sum(gelu(x*w+b), -1) on x[8192,1024] fp32."""

    name = "affine_gelu_rowsum_f32_8192x1024"
    dtype = "f32"
    rows, cols = 8192, 1024

    def algorithmic_bytes(self):
        return self.rows * self.cols * 4 + 2 * self.cols * 4 + self.rows * 4  # 33,595,392

    def load_host(self, seed):
        from oracle import inputs

        self.host = inputs.c1(self.rows, self.cols, seed=seed)
        return self.host

    def setup(self, device, seed, n_sets=8):
        d = self.load_host(seed)
        self.w, self.b = d["w"].to(device), d["b"].to(device)
        x = d["x"].to(device)
        # 32 MiB fits in L2: rotate over 8 copies (256 MiB) so every step reads from HBM
        self.xs = [x] + [x.clone() for _ in range(n_sets - 1)]

    def args(self, i):
        return (self.xs[i % len(self.xs)], self.w, self.b)

    def graph(self):
        import torch.nn.functional as F

        return lambda x, w, b: F.gelu(x * w + b).sum(-1)

    def prebuilt(self, x, w, b):
        from inductor_x_b200 import ops

        return ops.affine_gelu_rowsum(x, w, b)

    def e2e_setup(self, device):
        self.h_x = self.host["x"].pin_memory()
        self.h_o = torch.empty(self.rows).pin_memory()
        self.d_x = torch.empty_like(self.xs[0])

    def e2e_step(self):
        self.d_x.copy_(self.h_x, non_blocking=True)
        self.h_o.copy_(self.op(self.d_x, self.w, self.b), non_blocking=True)
        return self.h_x.numel() * 4, self.rows * 4

    def cpu_sample(self, rows=8192):
        import torch.nn.functional as F

        d = self.host
        x = d["x"][:rows]
        fn = lambda: F.gelu(x * d["w"] + d["b"]).sum(-1)
        return fn, rows * self.cols * 4 + 2 * self.cols * 4 + rows * 4, f"{rows} of {self.rows} rows, eager PyTorch ops"


class PermutedAmax(Workload):
    """configs[2] part 1: amax over dim 1 of x[64,128,256,64].permute(0,2,1,3), fp16."""

    name = "permuted_amax_f16_64x128x256x64"
    dtype = "f16"
    shape = (64, 128, 256, 64)
    shard_axis = "outer slabs"

    def algorithmic_bytes(self):
        a, b, c, d = self.shape
        return a * b * c * d * 2 + a * b * d * 2  # 269,484,032

    def load_host(self, seed):
        from oracle import inputs

        self.host = inputs.c3a(self.shape, seed=seed)["x"]
        return self.host

    def setup(self, device, seed, n_sets=3):
        x = self.load_host(seed)
        xd = x.to(device)
        self.xs = [xd] + [xd.clone() for _ in range(n_sets - 1)]

    def args(self, i):
        return (self.xs[i % len(self.xs)],)

    def graph(self):
        return lambda t: t.permute(0, 2, 1, 3).amax(1)

    def prebuilt(self, x):
        from inductor_x_b200 import ops

        a, b, c, d = x.shape
        return ops.outer_reduce(x.view(a * b, c, d), "amax", rsplit=1)

    def out_elems(self):
        a, b, c, d = self.shape
        return a * b * d

    def e2e_setup(self, device):
        self.h_x = self.host.pin_memory()
        self.d_x = torch.empty_like(self.xs[0])
        self.h_o = torch.empty(self.out_elems(), dtype=torch.float16).pin_memory()

    def e2e_step(self):
        self.d_x.copy_(self.h_x, non_blocking=True)
        self.h_o.copy_(self.op(self.d_x).reshape(-1), non_blocking=True)
        return self.h_x.numel() * 2, self.h_o.numel() * 2

    def cpu_sample(self, slabs=8):
        x = self.host[:slabs]
        fn = lambda: x.permute(0, 2, 1, 3).amax(1)
        _, b, c, d = self.shape
        return fn, slabs * b * c * d * 2 + slabs * b * d * 2, f"{slabs} of {self.shape[0]} outer slabs, eager PyTorch"


class PermutedSum(PermutedAmax):
    """configs[2] part 2: sum over dim 3 of the same permuted view -> [64,256,128]."""

    name = "permuted_sum_f16_64x128x256x64"

    def algorithmic_bytes(self):
        a, b, c, d = self.shape
        return a * b * c * d * 2 + a * b * c * 2  # 272,629,760

    def graph(self):
        return lambda t: t.permute(0, 2, 1, 3).sum(3)

    def prebuilt(self, x):
        from inductor_x_b200 import ops

        a, b, c, d = x.shape
        return ops.short_row_reduce(x, "sum", (c * b, 1, b))

    def out_elems(self):
        a, b, c, d = self.shape
        return a * b * c

    def cpu_sample(self, slabs=8):
        x = self.host[:slabs]
        fn = lambda: x.permute(0, 2, 1, 3).sum(3)
        _, b, c, d = self.shape
        return fn, slabs * b * c * d * 2 + slabs * b * c * 2, f"{slabs} of {self.shape[0]} outer slabs, eager PyTorch"


class IndexSelect(Workload):
    """configs[2] part 3: index_select of 262144 rows from a [2^20,128] fp16 table."""

    name = "index_select_f16_1Mx128_262144"
    dtype = "u8"  # bytes are moved, not computed on
    n_rows, dim, n_idx = 1 << 20, 128, 262144
    shard_axis = "index rows (table replicated)"

    def algorithmic_bytes(self):
        return self.n_idx * 8 + 2 * self.n_idx * self.dim * 2  # 136,314,880

    def load_host(self, seed):
        from oracle import inputs

        self.host = inputs.c3b(self.n_rows, self.dim, self.n_idx, seed=seed)
        return self.host

    def setup(self, device, seed, n_sets=4):
        d = self.load_host(seed)
        self.table = d["table"].to(device)  # 256 MiB: larger than L2
        g = torch.Generator().manual_seed(seed + 1000)
        # different random index sets per step so rows are not L2-resident from the last step
        self.xs = [d["idx"].to(device)] + [
            torch.randint(0, self.n_rows, (self.n_idx,), generator=g).to(device) for _ in range(n_sets - 1)]

    def args(self, i):
        return (self.table, self.xs[i % len(self.xs)])

    def graph(self):
        return lambda t, i: t.index_select(0, i)

    def prebuilt(self, table, idx):
        from inductor_x_b200 import ops

        return ops.index_select_rows(table, idx, check_bounds=False)

    def e2e_setup(self, device):
        self.h_idx = self.host["idx"].pin_memory()
        self.d_idx = torch.empty_like(self.xs[0])
        self.h_o = torch.empty(self.n_idx, self.dim, dtype=torch.float16).pin_memory()

    def e2e_step(self):
        self.d_idx.copy_(self.h_idx, non_blocking=True)
        self.h_o.copy_(self.op(self.table, self.d_idx), non_blocking=True)
        return self.n_idx * 8, self.h_o.numel() * 2

    def cpu_sample(self):
        d = self.host
        fn = lambda: d["table"].index_select(0, d["idx"])
        return fn, self.algorithmic_bytes(), "full workload, torch.index_select on CPU"


class FusedAttention(Workload):
    """configs[3]: causal attention, B=8, H=32, S=4096, D=128, bf16 (batch sharded over GPUs).
    The compiled graph is the pattern written out - matmul, scale, causal mask, softmax,
    matmul - which the backend's FX pattern turns into the tcgen05 kernel."""

    name = "fused_attention_bf16_b8_h32_s4096_d128_causal"
    dtype = "bf16"
    B, H, S, D = 8, 32, 4096, 128
    metric = "fused-attention TFLOP/s"
    unit = "TFLOP/s"
    bound = "tensor"
    n_out_sets = 1
    shard_axis = "batch"

    def flops(self):
        # causal-half convention: 4 * B * H * S^2 * D / 2
        return 4 * self.B * self.H * self.S * self.S * self.D // 2

    def algorithmic_bytes(self):
        return 4 * self.B * self.H * self.S * self.D * 2

    def load_host(self, seed):
        from oracle import inputs

        self.host = inputs.c4(self.B, self.H, self.S, self.D, seed=seed)
        self.scale = self.host["scale"]
        return self.host

    def setup(self, device, seed, n_sets=1):
        d = self.load_host(seed)
        self.q, self.k, self.v = (d[n].to(device) for n in "qkv")
        self.scale = d["scale"]
        self.xs = [self.q]

    def args(self, i):
        return (self.q, self.k, self.v)

    def graph(self):
        scale = self.scale

        def attention(q, k, v):
            n = q.shape[-2]
            keep = torch.ones(n, n, dtype=torch.bool, device=q.device).tril()
            s = torch.matmul(q, k.transpose(-2, -1)) * scale
            s = s.masked_fill(~keep, float("-inf"))
            return torch.matmul(torch.softmax(s, dim=-1), v)

        return attention

    def prebuilt(self, q, k, v):
        from inductor_x_b200 import ops

        return ops.fused_attention(q, k, v, self.scale, causal=True)

    def e2e_setup(self, device):
        self.h = [self.host[n].pin_memory() for n in "qkv"]
        self.d = [torch.empty_like(self.q) for _ in range(3)]
        self.h_o = torch.empty_like(self.h[0]).pin_memory()

    def e2e_step(self):
        for dst, src in zip(self.d, self.h):
            dst.copy_(src, non_blocking=True)
        self.h_o.copy_(self.op(self.d[0], self.d[1], self.d[2]), non_blocking=True)
        return 3 * self.h[0].numel() * 2, self.h_o.numel() * 2

    def cpu_sample(self, heads=2):
        import torch.nn.functional as F

        q, k, v = (self.host[n][:1, :heads].float() for n in "qkv")
        fn = lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=self.scale)
        return fn, 4 * heads * self.S * self.S * self.D // 2, f"{heads} of {self.B * self.H} heads, CPU SDPA fp32"


class FusedAttentionTraining(FusedAttention):
    """Training step of configs[3]: forward and backward of the same literal causal graph with
    gradients required.  The joint-graph pattern replaces both halves: the forward kernel, then
    delta, dK/dV and dQ kernels (tcgen05).  FLOPs: 3.5 x the forward count (2 forward products
    + 5 backward products, causal halves) - the recomputed probabilities of the two backward
    kernels (7 products actually issued) are not counted."""

    name = "fused_attention_fwd_bwd_bf16_b8_h32_s4096_d128_causal"
    metric = "fused-attention training TFLOP/s (forward + backward)"
    graph_capture = False     # autograd runs the backward graph: timed as an enqueue loop

    def flops(self):
        return 7 * super().flops() // 2

    def algorithmic_bytes(self):
        return 8 * self.B * self.H * self.S * self.D * 2

    def setup(self, device, seed, n_sets=1):
        super().setup(device, seed, n_sets)
        for t in (self.q, self.k, self.v):
            t.requires_grad_(True)
        g = torch.Generator().manual_seed(100 + seed)
        self.dy = torch.randn(self.q.shape, generator=g).to(self.q.dtype).to(device)

    def op(self, q, k, v):
        out = self.compiled(q, k, v) if self.path == "compiled" else self.prebuilt(q, k, v)
        return (out,) + torch.autograd.grad(out, (q, k, v), self.dy)

    def prebuilt(self, q, k, v):
        from inductor_x_b200.fusion_attention_graph import b200_fusion_attention_graph

        return b200_fusion_attention_graph(q, k, v, self.H, "BNSD", scale=1.0 / self.scale, sparse_mode=3)[0]

    def e2e_setup(self, device):
        self.h = [self.host[n].pin_memory() for n in "qkv"]
        self.h_dy = self.dy.cpu().pin_memory()
        self.d = [torch.empty_like(self.q).requires_grad_(True) for _ in range(3)]
        self.h_g = [torch.empty_like(self.h[0]).pin_memory() for _ in range(3)]

    def e2e_step(self):
        with torch.no_grad():
            for dst, src in zip(self.d, self.h):
                dst.copy_(src, non_blocking=True)
            self.dy.copy_(self.h_dy, non_blocking=True)
        res = self.op(*self.d)
        for dst, src in zip(self.h_g, res[1:]):
            dst.copy_(src, non_blocking=True)
        return 4 * self.h[0].numel() * 2, 3 * self.h[0].numel() * 2

    def cpu_sample(self, heads=1):
        q, k, v = (self.host[n][:1, :heads].float().requires_grad_(True) for n in "qkv")
        dy = torch.ones_like(q)
        keep = torch.ones(self.S, self.S, dtype=torch.bool).tril()

        def fn():
            s = (q @ k.transpose(-1, -2) * self.scale).masked_fill(~keep, float("-inf"))
            return torch.autograd.grad(torch.softmax(s, -1) @ v, (q, k, v), dy)

        return fn, 7 * (4 * heads * self.S * self.S * self.D // 2) // 2, \
            f"{heads} of {self.B * self.H} heads, eager fp32 attention + autograd on CPU"


class LlamaLayer(Workload):
    """configs[4]: Llama-style decoder layer through torch.compile (this backend): hidden 4096,
    32 heads x 128, SwiGLU 11008, batch 16 x seq 2048, bf16.  GEMMs stay extern (cuBLAS) as in
    stock Inductor; every other kernel is a template instantiation or the attention kernel."""

    name = "llama_layer_bf16_b16_s2048_h4096_ffn11008"
    dtype = "bf16"
    B, S, hidden, heads, ffn = 16, 2048, 4096, 32, 11008
    metric = "graph throughput (tokens/s); ms_per_step is the graph latency"
    unit = "tokens/s"
    bound = "tensor"
    n_out_sets = 1
    shard_axis = "batch"
    graph_capture = False     # library GEMMs pick workspaces at run time: timed as an enqueue loop

    def flops(self):
        t = self.B * self.S
        gemm = 2 * t * (4 * self.hidden * self.hidden + 3 * self.hidden * self.ffn)
        attn = 4 * self.B * self.heads * self.S * self.S * (self.hidden // self.heads) // 2
        return gemm + attn

    def algorithmic_bytes(self):
        return 2 * self.B * self.S * self.hidden * 2

    def load_host(self, seed):
        from oracle import inputs

        self.host = {"w": inputs.c5_weights(self.hidden, self.heads, self.ffn, seed=0),
                     "x": inputs.c5_input(self.B, self.S, self.hidden, seed=1 + seed)}
        return self.host

    def setup(self, device, seed, n_sets=1):
        from oracle import inputs

        d = self.load_host(seed)
        self.w = {k: v.to(device) for k, v in d["w"].items()}
        self.x = d["x"].to(device)
        cos, sin = inputs.rope_tables(self.S, self.hidden // self.heads)
        self.cos, self.sin = cos.to(device), sin.to(device)
        self.xs = [self.x]

    def args(self, i):
        return (self.x, self.cos, self.sin)

    def graph(self):
        from inductor_x_b200.llama_layer import decoder_layer

        return lambda x, cos, sin: decoder_layer(x, self.w, cos, sin, heads=self.heads)

    def prebuilt(self, x, cos, sin):
        raise SystemExit("the decoder layer has no prebuilt form: it is a torch.compile workload")

    def work(self):
        return self.B * self.S * 1e9      # tokens: value = tokens / s

    def e2e_setup(self, device):
        self.h_x = self.host["x"].pin_memory()
        self.d_x = torch.empty_like(self.x)
        self.h_o = torch.empty_like(self.h_x).pin_memory()

    def e2e_step(self):
        self.d_x.copy_(self.h_x, non_blocking=True)
        self.h_o.copy_(self.op(self.d_x, self.cos, self.sin), non_blocking=True)
        return self.h_x.numel() * 2, self.h_o.numel() * 2

    def cpu_sample(self, batch=1, seq=256):
        from oracle import graphs

        x = self.host["x"][:batch, :seq].contiguous()
        fn = lambda: graphs.llama_layer(x, self.host["w"], heads=self.heads, compute=torch.bfloat16)
        return fn, batch * seq, f"{batch} x {seq} of {self.B} x {self.S} tokens, eager PyTorch bf16 on CPU"


class CpMerge(Workload):
    """Ring-attention merge step (the reference's forward_update profile case,
    test/npu_indexing/written/test_attn_cp.py:241-252): (S, B, H, N) = (8192, 1, 6144, 48),
    bf16 attention outputs, fp32 [B, N, S, 8] statistics.  A kernel-library workload: its
    compiled form is covered by tests/test_compile_gpu.py at small size."""

    name = "cp_forward_update_bf16_s8192_h6144_n48"
    dtype = "bf16"
    S, B, H, N = 8192, 1, 6144, 48
    path = "prebuilt"
    KEYS = ("prev_attn_out", "prev_softmax_max", "prev_softmax_sum", "cur_attn_out", "cur_softmax_max",
            "cur_softmax_sum")

    def algorithmic_bytes(self):
        attn = self.S * self.B * self.H * 2
        stats = self.B * self.N * self.S * 8 * 4
        return 3 * attn + 6 * stats   # two attention reads + one write; four statistics reads + two writes

    def load_host(self, seed):
        from oracle import inputs

        self.host = inputs.cp_merge(self.S, self.B, self.H, self.N, seed=seed)
        return self.host

    def setup(self, device, seed, n_sets=2):
        d = self.load_host(seed)
        # two sets of ~240 MB of inputs each: more than L2 between consecutive steps
        self.xs = [[d[k].to(device) for k in self.KEYS]]
        for _ in range(n_sets - 1):
            self.xs.append([t.clone() for t in self.xs[0]])

    def bind(self, path):
        return super().bind("prebuilt")

    def args(self, i):
        return tuple(self.xs[i % len(self.xs)])

    def prebuilt(self, *tensors):
        from inductor_x_b200 import ops

        return ops.forward_update(*tensors)

    def e2e_setup(self, device):
        self.h_in = [self.host[k].pin_memory() for k in self.KEYS]
        self.d_in = [torch.empty_like(t) for t in self.xs[0]]
        self.h_o = torch.empty(self.S, self.B, self.H, dtype=torch.bfloat16).pin_memory()

    def e2e_step(self):
        for d, h in zip(self.d_in, self.h_in):
            d.copy_(h, non_blocking=True)
        o, _, _ = self.op(*self.d_in)
        self.h_o.copy_(o, non_blocking=True)
        return sum(t.numel() * t.element_size() for t in self.h_in), self.h_o.numel() * 2

    def cpu_sample(self):
        from oracle import graphs

        d = self.host
        fn = lambda: graphs.cp_forward_update(**d)
        return fn, self.algorithmic_bytes(), "full workload, eager PyTorch on CPU (the reference's forward_update)"


class RowCumsum(Workload):
    """cumsum along the last axis of x[16384, 4096] bf16: the row template's team-wide prefix scan
    (the reference leaves every cumsum to an extern kernel, inductor_x/lowering.py:235-245)."""

    name = "cumsum_lastdim_bf16_16384x4096"
    dtype = "bf16"
    rows, cols = 16384, 4096

    def algorithmic_bytes(self):
        return 2 * self.rows * self.cols * 2

    def load_host(self, seed):
        g = torch.Generator().manual_seed(seed)
        self.host = torch.randn(self.rows, self.cols, generator=g).bfloat16()
        return self.host

    def setup(self, device, seed, n_sets=3):
        x = self.load_host(seed).to(device)
        self.xs = [x] + [x.clone() for _ in range(n_sets - 1)]

    def args(self, i):
        return (self.xs[i % len(self.xs)],)

    def graph(self):
        return lambda t: torch.cumsum(t, -1)

    def prebuilt(self, x):
        raise SystemExit("the scan exists only in generated form")

    def e2e_setup(self, device):
        self.h_x = self.host.pin_memory()
        self.d_x = torch.empty_like(self.xs[0])
        self.h_o = torch.empty_like(self.h_x).pin_memory()

    def e2e_step(self):
        self.d_x.copy_(self.h_x, non_blocking=True)
        self.h_o.copy_(self.op(self.d_x), non_blocking=True)
        return self.h_x.numel() * 2, self.h_o.numel() * 2

    def cpu_sample(self, rows=1024):
        x = self.host[:rows].float()
        return (lambda: torch.cumsum(x, -1)), 2 * rows * self.cols * 2, f"{rows} of {self.rows} rows, torch.cumsum on CPU"


class PermutedPointwise(Workload):
    """x[8,8,512,128] fp16 -> (x.permute(0,2,1,3) + 1).contiguous(): a permuted pointwise copy whose
    innermost axis is kept (128-bit access on both sides).  64 copies of the tensor per step
    (a [64,8,8,512,128] batch) so that one step moves 1 GiB."""

    name = "permute_0213_f16_64x8x8x512x128"
    dtype = "f16"
    shape = (64 * 8, 8, 512, 128)
    perm = (0, 2, 1, 3)
    shard_axis = "batch"

    def algorithmic_bytes(self):
        n = 1
        for d in self.shape:
            n *= d
        return 2 * n * 2

    def load_host(self, seed):
        g = torch.Generator().manual_seed(seed)
        self.host = (torch.rand(*self.shape, generator=g) * 2 - 1).half()
        return self.host

    def setup(self, device, seed, n_sets=2):
        x = self.load_host(seed).to(device)
        self.xs = [x] + [x.clone() for _ in range(n_sets - 1)]

    def args(self, i):
        return (self.xs[i % len(self.xs)],)

    def graph(self):
        perm = self.perm
        return lambda t: (t.permute(*perm) + 1.0).contiguous()

    def prebuilt(self, x):
        raise SystemExit("permuted pointwise graphs exist only in compiled form")

    def e2e_setup(self, device):
        self.h_x = self.host.pin_memory()
        self.d_x = torch.empty_like(self.xs[0])
        self.h_o = torch.empty(self.host.numel(), dtype=torch.float16).pin_memory()

    def e2e_step(self):
        self.d_x.copy_(self.h_x, non_blocking=True)
        self.h_o.copy_(self.op(self.d_x).reshape(-1), non_blocking=True)
        return self.h_x.numel() * 2, self.h_o.numel() * 2

    def cpu_sample(self, n=32):
        x = self.host[:n]
        perm = self.perm
        fn = lambda: (x.permute(*perm) + 1.0).contiguous()
        return fn, 2 * x.numel() * 2, f"{n} of {self.shape[0]} outer slabs, eager PyTorch"


class TransposedPointwise(PermutedPointwise):
    """The same tensor with its two innermost axes swapped, (0,1,3,2): a true transpose - loads
    contiguous along one digit of the output index, stores along another."""

    name = "transpose_0132_f16_64x8x8x512x128"
    perm = (0, 1, 3, 2)


WORKLOADS = {
    "c2": SoftmaxLayerNorm, "c1": AffineGeluRowSum, "c3a_amax": PermutedAmax,
    "c3a_sum": PermutedSum, "c3b": IndexSelect, "c4": FusedAttention, "c4_train": FusedAttentionTraining,
    "c5": LlamaLayer, "cp": CpMerge, "perm": PermutedPointwise, "transpose": TransposedPointwise,
    "cumsum": RowCumsum,
}
#: configurations reported under `configs` after the headline: (key, steps per replay, replays floor)
SECONDARY = ("c1", "c3a_amax", "c3a_sum", "c3b", "perm", "transpose", "cumsum", "c4", "c4_train", "c5")


# ---------------------------------------------------------------------------- driver
def time_cpu(fn, min_seconds=2.0, max_iters=50):
    fn()
    fn()
    best, total, it = float("inf"), 0.0, 0
    while (total < min_seconds or it < 5) and it < max_iters:
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        best = min(best, dt)
        total += dt
        it += 1
    return best


def run_reference(args, wl_cls):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    wl = wl_cls()
    wl.load_host(0)  # host data only; no GPU is touched on this arm
    fn, nwork, sample = wl.cpu_sample()
    for _ in range(max(args.warmup, 1)):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    dt = (time.perf_counter() - t0) / args.steps
    scale = 1.0 if wl.unit == "tokens/s" else (1e12 if wl.bound == "tensor" else 1e9)
    val = nwork / dt / scale
    line = {
        "impl": "reference", "metric": wl.metric, "value": val, "unit": wl.unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype,
        "data": "synthetic",
        "config": {"workload": wl.name, "note": "eager PyTorch on host cores; the reference's own "
                   "ground truth (it asserts compiled == eager) - the reference itself needs an Ascend NPU"},
        "cpu_baseline": {"value": val, "unit": wl.unit, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


class Env:
    """Process-wide state of one bench run: rank, device, peaks, barrier, traffic table."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.device = torch.device("cuda", self.local_rank)
        self.peaks = measured_peaks()
        self.traffic = {}
        tpath = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(tpath):
            with open(tpath) as f:
                self.traffic = json.load(f)

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, value: float) -> float:
        if self.world == 1:
            return value
        import torch.distributed as dist

        t = torch.tensor([value], device=self.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())


def count_launches(fn):
    """Kernels of this package launched by ``fn()``: generated modules count their launches;
    the library's tensor-level wrappers launch one kernel per call."""
    from inductor_x_b200 import ops
    from inductor_x_b200.codegen import jit

    before = sum(k.launches for k in jit._loaded.values()) + ops.launch_count()
    fn()
    return sum(k.launches for k in jit._loaded.values()) + ops.launch_count() - before


def time_device(env: Env, wl: Workload, steps: int, warmup: int, use_graph: bool, min_seconds: float):
    """Device time of `steps` steps: the K launches are captured into one CUDA graph and the
    graph is replayed R times (R chosen so that the timed region lasts at least
    `min_seconds`), each replay bracketed by CUDA events on the launching stream.  A kernel of
    a few microseconds is thereby timed back to back on the device instead of at the pace
    Python can enqueue it.  Returns per-step times: median and mean over the replays."""
    for i in range(max(warmup, 3)):
        wl.step(i)
    env.barrier()
    launches_per_step = count_launches(lambda: wl.step(0))
    env.barrier()
    graph = None
    if use_graph and getattr(wl, "graph_capture", True):
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for i in range(steps):
                        wl.step(i)
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()  # one untimed replay
            env.barrier()
        except Exception as e:  # capture not possible: time the enqueue loop instead
            print(f"graph capture failed ({type(e).__name__}: {e}); timing the enqueue loop", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    def one_pass():
        if graph is not None:
            graph.replay()
        else:
            for i in range(steps):
                wl.step(i)

    # size the timed region from one probe pass
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    one_pass()
    p1.record()
    env.barrier()
    probe_ms = max(p0.elapsed_time(p1), 1e-3)
    replays = int(min(max(1, -(-min_seconds * 1e3 // probe_ms)), 2000))
    if env.world > 1:
        replays = int(env.max_over_ranks(float(replays)))
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
    t_wall0 = time.perf_counter()
    marks[0].record()
    for r in range(replays):
        one_pass()
        marks[r + 1].record()
    env.barrier()
    t_wall1 = time.perf_counter()
    per_replay = sorted(marks[r].elapsed_time(marks[r + 1]) for r in range(replays))
    total_ms = env.max_over_ranks(marks[0].elapsed_time(marks[replays]))
    return {
        "ms_per_step": total_ms / (replays * steps),
        "kernel_ms_avg": marks[0].elapsed_time(marks[replays]) / (replays * steps),
        "kernel_ms_median": per_replay[len(per_replay) // 2] / steps,
        "kernel_ms_min": per_replay[0] / steps,
        "replays": replays, "steps": steps, "launches_per_step": launches_per_step,
        "timed_region": ("one CUDA graph of the K launches, replayed" if graph is not None else "enqueue loop"),
        "wall": (t_wall0, t_wall1),
    }


def time_e2e(env: Env, wl: Workload, e2e_steps: int):
    """The same metric through the same call with HOST buffers: pinned host-to-device copies of
    the step's inputs and the device-to-host read of its result inside the timed region."""
    wl.e2e_setup(env.device)
    for _ in range(2):
        wl.e2e_step()
    env.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        h2d, d2h = wl.e2e_step()
    e1.record()
    env.barrier()
    ms = env.max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
    return {"value": env.world * wl.work() / (ms * 1e-3) / 1e9, "unit": wl.unit,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms}


def roofline_of(env: Env, wl: Workload, timing: dict):
    tensor = wl.bound == "tensor"
    ms = timing["kernel_ms_median"]
    work = wl.flops() / 1e3 if tensor else wl.algorithmic_bytes()
    achieved = work / (ms * 1e-3) / 1e9
    # The tensor peak is the cuBLAS figure measured the same way the kernel is: back to back for
    # a quarter of a second or more the part sits at its power cap and the sustained figure
    # applies; a shorter region is compared with the burst figure.
    region_s = timing["kernel_ms_avg"] * timing["steps"] * timing["replays"] * 1e-3
    sustained = tensor and region_s >= 0.25
    peak = (env.peaks["bf16_tflops_sustained"] if sustained else env.peaks["bf16_tflops"]) if tensor \
        else env.peaks["hbm_gbs"]
    traffic = env.traffic.get(f"{wl.name}:{wl.path}", env.traffic.get(wl.name) if wl.path == "prebuilt" else None)
    out = {"bound": "tensor" if tensor else "hbm", "achieved": achieved, "peak": peak,
           "unit": "TFLOP/s" if tensor else "GB/s", "frac": achieved / peak, "traffic": traffic,
           "peak_source": env.peaks["source"], "kernel_ms_avg": timing["kernel_ms_avg"],
           "kernel_ms_median": ms, "kernel_ms_min": timing["kernel_ms_min"],
           "frac_of_nominal": achieved / (2250.0 if tensor else 8000.0)}
    if tensor:
        out["peak_kind"] = "sustained" if sustained else "burst"
        out["frac_of_burst"] = achieved / env.peaks["bf16_tflops"]
    if traffic and not tensor:
        # bytes that actually crossed the DRAM interface (one ncu capture) over the same time: shows
        # how much of `frac` the L2 contributed
        out["dram_frac"] = traffic / (ms * 1e-3) / 1e9 / peak
    return out


def run_config(env: Env, key: str, args, path: str, steps: int, min_seconds: float, e2e_steps: int,
               batch_div: int = 1):
    """Set up, time and tear down one configuration; returns its entry for `configs`."""
    wl = WORKLOADS[key]()
    if batch_div > 1:
        wl.B = max(1, wl.B // batch_div)
    wl.setup(env.device, seed=env.rank)
    wl.bind(path)
    timing = time_device(env, wl, steps, 3, not args.no_graph, min_seconds)
    e2e = time_e2e(env, wl, e2e_steps)
    value = env.world * wl.work() / (timing["ms_per_step"] * 1e-3) / 1e9
    entry = {"workload": wl.name, "path": path_name(wl.path), "dtype": wl.dtype, "metric": wl.metric,
             "value": value, "unit": wl.unit, "ms_per_step": timing["ms_per_step"],
             "steps": timing["steps"], "replays": timing["replays"],
             "gpu_launches_per_step": timing["launches_per_step"], "timed_region": timing["timed_region"],
             "roofline": roofline_of(env, wl, timing), "e2e": e2e}
    if key == "c5":
        entry["roofline"] = None          # a graph of many kernels: latency and tokens/s are the figures
        entry["effective_tflops"] = wl.flops() / (timing["ms_per_step"] * 1e-3) / 1e12
    del wl
    torch.cuda.empty_cache()
    return entry


def path_name(path: str) -> str:
    return "torch.compile -> generated kernels" if path == "compiled" else "prebuilt kernel library entry point"


def sharded_configs(env: Env, args):
    """N > 1: a FIXED global batch cut along its outer axis (strong scaling), and the all-gather
    of the sharded output where a consumer needs the full tensor."""
    import torch.distributed as dist

    from inductor_x_b200 import sharding

    out = []
    # fused attention, global batch 8 split over the ranks
    if FusedAttention.B % env.world == 0:
        e = run_config(env, "c4", args, args.path, steps=4, min_seconds=0.4, e2e_steps=1, batch_div=env.world)
        e["scaling"] = "strong"
        e["global_batch"] = FusedAttention.B
        out.append(e)
    # softmax -> LayerNorm, 16384 rows split over the ranks; every rank's kernel writes its rows
    # into its slot of the full output and the all-gather runs in place
    wl = SoftmaxLayerNorm()
    lo, hi = sharding.shard_bounds(wl.rows, env.world, env.rank)
    full_rows = wl.rows
    wl.rows = hi - lo
    wl.setup(env.device, seed=0, n_sets=2)
    wl.rows = full_rows
    wl.bind(args.path)
    shard = sharding.OuterAxisShard(env.world, env.rank, dist.group.WORLD)
    full = torch.empty(full_rows, wl.cols, dtype=torch.bfloat16, device=env.device)
    fn = lambda x, out: wl.op_into(out, x)
    for _ in range(3):
        shard.run_local(fn, wl.xs[0], full, gather=True)
    env.barrier()
    # kernel: K launches captured in one CUDA graph and replayed (a 4096-row shard runs for ~20 us,
    # far below what Python needs to enqueue it); collective: back-to-back all-gathers between events
    reps = 20
    graph = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(reps):
                    shard.run_local(fn, wl.xs[i % 2], full, gather=False)
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
    except Exception as e:
        print(f"graph capture of the sharded kernel failed ({type(e).__name__}: {e}); timing the enqueue loop",
              file=sys.stderr)
        graph = None
        torch.cuda.synchronize()
    env.barrier()
    times = []
    for _ in range(7):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if graph is not None:
            graph.replay()
        else:
            for i in range(reps):
                shard.run_local(fn, wl.xs[i % 2], full, gather=False)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / reps)
    k_ms = env.max_over_ranks(sorted(times)[len(times) // 2])
    env.barrier()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(reps):
        shard.gather(full)
    g1.record()
    torch.cuda.synchronize()
    c_ms = env.max_over_ranks(g0.elapsed_time(g1) / reps)
    nbytes = 2 * full_rows * wl.cols * 2
    out.append({"workload": wl.name, "path": path_name(wl.path), "scaling": "strong", "global_rows": full_rows,
                "kernel_ms": k_ms, "all_gather_ms": c_ms, "value": nbytes / ((k_ms + c_ms) * 1e-3) / 1e9,
                "kernel_timed_region": "one CUDA graph of 20 launches, replayed" if graph is not None else "enqueue loop",
                "unit": "GB/s", "gathered_bytes": full_rows * wl.cols * 2,
                "all_gather_busbw_gbs": full_rows * wl.cols * 2 * (env.world - 1) / env.world / (c_ms * 1e-3) / 1e9})
    return out


def host_copy_ceiling(env: Env, nbytes: int = 128 << 20):
    """Pinned host<->device copy bandwidth of this rank with all ranks copying at once: the
    ceiling of any end-to-end figure."""
    h = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d = torch.empty(nbytes, dtype=torch.uint8, device=env.device)
    out = {}
    for name, (dst, src) in (("h2d", (d, h)), ("d2h", (h, d))):
        dst.copy_(src, non_blocking=True)
        env.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(4):
            dst.copy_(src, non_blocking=True)
        e1.record()
        env.barrier()
        out[f"{name}_gbs_per_rank"] = 4 * nbytes / (env.max_over_ranks(e0.elapsed_time(e1)) * 1e-3) / 1e9
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--min-seconds", type=float, default=0.6,
                    help="the K-step graph is replayed until the timed region lasts this long")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="headline only: skip the other configurations")
    ap.add_argument("--no-graph", action="store_true", help="time the Python enqueue loop instead of a CUDA graph")
    ap.add_argument("--prebuilt", action="store_true",
                    help="time the hand-instantiated entry points of the kernel library instead of the "
                         "graphs compiled through torch.compile")
    ap.add_argument("--compiled", action="store_true", help="(default) kept for old command lines")
    ap.add_argument("--c4-batch", type=int, default=0,
                    help="override the attention batch (profiling captures on a smaller case)")
    args = ap.parse_args()
    args.path = "prebuilt" if args.prebuilt else "compiled"
    wl_cls = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference(args, wl_cls)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the backend has no CPU path")
    env = Env()
    torch.cuda.set_device(env.local_rank)
    import torch.distributed as dist

    if env.world > 1:
        dist.init_process_group("nccl", device_id=env.device)

    from inductor_x_b200 import runtime as rt

    rt.load()
    wl = wl_cls()
    if args.c4_batch > 0 and isinstance(wl, FusedAttention):
        wl.B = args.c4_batch
        wl.name = wl.name.replace("_b8_", f"_b{args.c4_batch}_")
    wl.setup(env.device, seed=env.rank)  # each rank owns a different shard of the global batch
    wl.bind(args.path)
    if isinstance(wl, SoftmaxLayerNorm):
        # every rank drives its own pinned staging pair; with several ranks on one host the copy
        # engines and the host memory system are shared, and fewer, larger chunks waste less
        wl.e2e_chunks = {1: 8, 2: 4}.get(env.world, 2)

    sampler = ClockSampler(env.local_rank)
    if env.rank == 0:
        sampler.start()

    timing = time_device(env, wl, args.steps, args.warmup, not args.no_graph, args.min_seconds)
    value = env.world * wl.work() / (timing["ms_per_step"] * 1e-3) / 1e9
    e2e = time_e2e(env, wl, args.e2e_steps)
    if env.rank == 0:
        sampler.stop_flag.set()
        sampler.join(timeout=2)
    clocks = sampler.summary(*timing["wall"]) if env.rank == 0 else None
    roof = roofline_of(env, wl, timing)
    if isinstance(wl, LlamaLayer):
        roof = {"bound": "tensor", "achieved": wl.flops() / (timing["kernel_ms_median"] * 1e-3) / 1e12,
                "peak": env.peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": wl.flops() / (timing["kernel_ms_median"] * 1e-3) / 1e12 / env.peaks["bf16_tflops_sustained"],
                "traffic": None, "peak_source": env.peaks["source"],
                "note": "whole graph (library GEMMs included) against the sustained GEMM figure"}

    cpu = None
    if env.rank == 0 and env.world == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        fn, cwork, sample = wl.cpu_sample()
        best = time_cpu(fn)
        scale = 1.0 if wl.unit == "tokens/s" else (1e12 if wl.bound == "tensor" else 1e9)
        cpu = {"value": cwork / best / scale, "unit": wl.unit, "cores": torch.get_num_threads(),
               "kind": "port", "sample": sample + f"; best of >=5, {best * 1e3:.2f} ms"}

    headline_name, headline_path, headline_dtype = wl.name, wl.path, wl.dtype
    headline_metric, headline_unit, headline_sets = wl.metric, wl.unit, wl.sets()
    headline_bytes, shard_axis = wl.algorithmic_bytes(), wl.shard_axis
    del wl
    torch.cuda.empty_cache()

    configs = []
    if not args.no_configs and args.workload == "c2":
        if env.world == 1:
            for key in SECONDARY:
                try:
                    steps = {"c4": 4, "c4_train": 2, "c5": 3}.get(key, 40)
                    configs.append(run_config(env, key, args,
                                              args.path if key not in ("c5", "perm", "transpose", "cumsum") else "compiled",
                                              steps=steps, min_seconds=0.3, e2e_steps=2))
                except Exception as e:      # one configuration failing must not lose the line
                    configs.append({"workload": key, "error": f"{type(e).__name__}: {e}"[:300]})
        else:
            try:
                configs = sharded_configs(env, args)
            except Exception as e:
                configs = [{"workload": "sharded", "error": f"{type(e).__name__}: {e}"[:300]}]
    ceiling = host_copy_ceiling(env)

    if env.rank == 0:
        line = {
            "metric": headline_metric, "value": value, "unit": headline_unit,
            "n_gpus": env.world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": timing["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": headline_dtype,
            "data": "synthetic",
            "config": {"workload": headline_name, "algorithmic_bytes_per_step": headline_bytes,
                       "l2": "working set per step exceeds the 126 MB L2 and steps rotate over "
                             f"{headline_sets} distinct input sets and 3 output blocks",
                       "sharding": f"{shard_axis} split over {env.world} GPU(s), no collective",
                       "path": path_name(headline_path),
                       "timed_region": timing["timed_region"], "replays": timing["replays"]},
            "roofline": roof,
            "cpu_baseline": cpu,
            "e2e": {**e2e, **ceiling},
            "gpu_launches": timing["launches_per_step"] * timing["steps"] * timing["replays"],
            "clocks": clocks,
            "configs": configs,
        }
        print(json.dumps(line), flush=True)
    if env.world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
