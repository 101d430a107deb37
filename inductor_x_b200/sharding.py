"""Outer-axis sharding over the GPUs of one box.

Every kernel family of this backend is independent along its outermost kept axis (rows of a
row kernel, outer slabs of an outer reduction, gathered rows, attention batch) - the axis
the reference splits over its vector cores (``inductor_x/codegen/split_tiling.py:46-75``).
Across GPUs the same axis is cut into contiguous chunks, one per rank, with no collective on
the data path.  Only when a consumer needs the whole tensor is the result gathered, and
then in place: the local kernel writes its chunk straight into its slot of the gather
buffer, so ``all_gather_into_tensor`` moves each byte over NVLink exactly once and no staging
copy exists.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous chunk [start, stop) of ``n`` items owned by ``rank``; the first
    ``n % world`` ranks get one extra item."""
    if world <= 0 or not (0 <= rank < world) or n < 0:
        raise ValueError(f"bad shard request n={n} world={world} rank={rank}")
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def even_shard(n: int, world: int) -> int:
    """Chunk size when ``n`` divides evenly (required by the in-place gather)."""
    if n % world != 0:
        raise ValueError(f"outer extent {n} is not a multiple of the world size {world}")
    return n // world


class OuterAxisShard:
    """Runs ``fn(local_input_chunk, out=local_output_slot)`` on this rank's chunk of the outer
    axis and, on request, gathers the full output in place."""

    def __init__(self, world: Optional[int] = None, rank: Optional[int] = None, group=None):
        self.group = group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)

    def local(self, full: torch.Tensor) -> torch.Tensor:
        a, b = shard_bounds(full.shape[0], self.world, self.rank)
        return full[a:b]

    def slot(self, full_out: torch.Tensor) -> torch.Tensor:
        """This rank's rows of a full-size output buffer (the extent must divide evenly)."""
        chunk = even_shard(full_out.shape[0], self.world)
        return full_out[self.rank * chunk:(self.rank + 1) * chunk]

    def run_local(self, fn: Callable, local_input: torch.Tensor, full_out: torch.Tensor,
                  gather: bool = False) -> torch.Tensor:
        """For a rank that holds only its own chunk of the input: ``fn(local_input, out=slot)``
        writes straight into this rank's slot of ``full_out``; with ``gather`` the other ranks'
        slots are then filled in place."""
        fn(local_input, out=self.slot(full_out))
        if gather:
            self.gather(full_out)
        return full_out

    def gather(self, full_out: torch.Tensor) -> torch.Tensor:
        """In-place all-gather: every rank's slot of ``full_out`` travels once over NVLink."""
        if self.world > 1:
            dist.all_gather_into_tensor(full_out, self.slot(full_out), group=self.group)
        return full_out

    def run(self, fn: Callable, full_input: torch.Tensor, out_shape_per_item: Tuple[int, ...],
            out_dtype: torch.dtype, gather: bool = False) -> torch.Tensor:
        n = full_input.shape[0]
        if gather:
            chunk = even_shard(n, self.world)
            full_out = torch.empty((n, *out_shape_per_item), dtype=out_dtype, device=full_input.device)
            slot = full_out[self.rank * chunk:(self.rank + 1) * chunk]
            fn(self.local(full_input), out=slot)          # written in place, no staging copy
            if self.world > 1:
                dist.all_gather_into_tensor(full_out, slot, group=self.group)
            return full_out
        a, b = shard_bounds(n, self.world, self.rank)
        out = torch.empty((b - a, *out_shape_per_item), dtype=out_dtype, device=full_input.device)
        fn(full_input[a:b], out=out)
        return out
