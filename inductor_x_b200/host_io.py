"""Host-buffer entry for row-sharded kernels: pinned host input -> device -> kernel ->
pinned host output, with the three stages overlapped chunk by chunk.

A caller that holds its tensors in host memory pays PCIe both ways; done naively (copy in,
run, copy out) the link is used in one direction at a time.  Here the outer axis is cut into
chunks and three streams work as a pipeline - chunk i+1 is uploaded while chunk i computes
and chunk i-1 is downloaded - so the link carries traffic in both directions at once.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch


class HostRowPipeline:
    """Reusable pipeline over the leading axis of one input / one output tensor.

    ``kernel(dev_in_chunk, out=dev_out_chunk)`` must enqueue on the current stream and
    treat chunks independently (every kernel family of this backend does, along its outer
    axis)."""

    def __init__(self, device, in_shape, in_dtype, out_shape, out_dtype, chunks: int = 8):
        self.device = torch.device(device)
        n = in_shape[0]
        if out_shape[0] != n:
            raise ValueError("input and output must share the outer extent")
        self.chunks = max(1, min(chunks, n))
        self.bounds = [(n * c // self.chunks, n * (c + 1) // self.chunks) for c in range(self.chunks)]
        self.d_in = torch.empty(in_shape, dtype=in_dtype, device=self.device)
        self.d_out = torch.empty(out_shape, dtype=out_dtype, device=self.device)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.ev_in = [torch.cuda.Event() for _ in range(self.chunks)]
        self.ev_k = [torch.cuda.Event() for _ in range(self.chunks)]

    def run(self, h_in: torch.Tensor, kernel: Callable, h_out: torch.Tensor) -> torch.Tensor:
        if not (h_in.is_pinned() and h_out.is_pinned()):
            raise ValueError("host buffers must be pinned for asynchronous copies")
        cur = torch.cuda.current_stream(self.device)
        # the staging buffers may still be in use by the previous call
        self.s_in.wait_stream(cur)
        self.s_in.wait_stream(self.s_out)
        for c, (a, b) in enumerate(self.bounds):
            with torch.cuda.stream(self.s_in):
                self.d_in[a:b].copy_(h_in[a:b], non_blocking=True)
                self.ev_in[c].record(self.s_in)
            cur.wait_event(self.ev_in[c])
            kernel(self.d_in[a:b], out=self.d_out[a:b])
            self.ev_k[c].record(cur)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_k[c])
                h_out[a:b].copy_(self.d_out[a:b], non_blocking=True)
        cur.wait_stream(self.s_out)
        return h_out
