"""Launch-configuration chooser for generated kernels.

Stands where the reference decides its split axis, tiling axes and tile sizes
(``SplitTiling.select_split_axis`` / ``select_tiling_axis`` / ``decide_nblocks_xblock``,
``inductor_x/codegen/split_tiling.py:46-182``; ``TileGenerator``,
``inductor_x/codegen/tile_generator.py:10-136``; ``triton_config_npu_index``,
``inductor_x/npu_triton_heuristics.py:467-544``).  On B200 the questions become:

* which template family a fused group maps to (pointwise / persistent row / looped),
* how many threads cooperate on a row and how many 128-bit vectors each holds,
* how wide the per-thread vector of a pointwise kernel is.

The split ("grid") axis is always the kept outer axis: CTAs are persistent over it, so no
XBLOCK/NBLOCKS arithmetic is needed, and the tiling axis is the stride-1 axis by
construction of the templates.
"""
from __future__ import annotations

import dataclasses
from typing import Iterable, Optional

import torch

from .. import config

# (team, vpt) pairs, same list as the prebuilt library dispatches over (csrc/host.h)
ROW_PAIRS = [(32, 1), (32, 2), (32, 4), (64, 4), (128, 2), (128, 4), (256, 2), (256, 4),
             (512, 2), (512, 4), (1024, 4), (1024, 8)]


@dataclasses.dataclass(frozen=True)
class RowConfig:
    team: int      # threads cooperating on one row
    teams: int     # rows processed concurrently by one CTA
    vpt: int       # 128-bit vectors per thread
    vec: int       # elements per vector

    @property
    def elems_per_thread(self) -> int:
        return self.vpt * self.vec

    @property
    def capacity(self) -> int:
        return self.team * self.vpt * self.vec


def narrowest_dtype(dtypes: Iterable[torch.dtype]) -> torch.dtype:
    """The storage type that fixes the vector width: the narrowest floating operand."""
    best = None
    for d in dtypes:
        if d not in config.BYTES_PER_ELEMENT:
            continue
        if best is None or config.byte_per_numel(d) < config.byte_per_numel(best):
            best = d
    return best or torch.float32


def choose_row_config(rnumel: int, dtype: torch.dtype, max_vpt: int = 4) -> Optional[RowConfig]:
    """Smallest team that covers a row of ``rnumel`` elements of ``dtype`` with at most
    ``max_vpt`` vectors per thread (generated bodies keep several fp32 copies of the row in
    registers, hence the tighter default than the prebuilt bodies).  None if the row does
    not fit on chip."""
    vec = max(config.get_aligned_numel(dtype), 1)
    vec = min(vec, 8)
    nvec = -(-rnumel // vec)
    best = None
    for team, vpt in ROW_PAIRS:
        if vpt > max_vpt and not (team == 1024 and vpt == 8):
            continue
        cap = team * vpt
        if cap < nvec:
            continue
        if best is None or cap < best[0] * best[1]:
            best = (team, vpt)
    if best is None:
        return None
    team, vpt = best
    return RowConfig(team=team, teams=max(1, 256 // team), vpt=vpt, vec=vec)


def choose_pointwise_vec(dtypes: Iterable[torch.dtype]) -> int:
    """Elements per thread of a pointwise kernel: one 128-bit access of the narrowest
    operand, at least 4."""
    d = narrowest_dtype(dtypes)
    return max(4, min(8, config.get_aligned_numel(d)))


def should_use_persistent_reduction(rnumel, dtype: torch.dtype) -> bool:
    """Rows are held on chip whenever they fit (the reference's bound is 1024 elements,
    ``inductor_x/codegen/triton.py:401-424``)."""
    try:
        r = int(rnumel)
    except (TypeError, ValueError):
        return False
    return choose_row_config(r, dtype) is not None
