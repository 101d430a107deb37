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

@dataclasses.dataclass(frozen=True)
class RowConfig:
    team: int          # threads cooperating on one row
    teams: int         # rows processed concurrently by one CTA
    vpt: int           # 128-bit vectors per thread
    vec: int           # elements per vector
    min_ctas: int = 1  # resident CTAs per SM the register allocation is bounded for
    prefetch: int = 0  # rows ahead whose streamed operands are prefetched into L2

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


MAX_TEAM = 1024
MIN_TEAM = 8          # teams narrower than a warp serve rows of a few vectors
MAX_VPT = 32         # beyond 8 the row no longer fits the register file and spills: slow but correct
MAX_PERSISTENT_VPT = 8   # static rows longer than MAX_TEAM x this many vectors are walked in chunks


def choose_row_config(rnumel: int, dtype: torch.dtype, rows: Optional[int] = None,
                      target_vpt: int = 2) -> Optional[RowConfig]:
    """Launch shape of a generated persistent-row kernel.

    A generated body keeps several fp32 copies of its part of the row live, so the row is
    spread thin: ``target_vpt`` vectors per thread over the smallest power-of-two team
    that covers it (measured on the softmax->LayerNorm chain at 4096 bf16 columns: 256
    threads x 2 vectors ran 1.2-2x faster than 128 x 4).  Only rows longer than 1024
    threads x ``target_vpt`` vectors take more per thread, and rows of a few vectors get
    teams of 8 or 16 lanes so that a warp works on several rows at once.  CTAs hold 128 threads or one
    team, whichever is larger, and the register allocation is bounded for 1024 resident
    threads per SM (the module loader relaxes the bound if that makes the body spill).
    Rows that are streamed long enough get an L2 prefetch two rows ahead.  None if the
    row does not fit on chip."""
    vec = min(max(config.get_aligned_numel(dtype), 1), 8)
    nvec = -(-rnumel // vec)
    if nvec > MAX_TEAM * MAX_VPT:
        return None
    vpt = target_vpt
    team = MIN_TEAM
    while team < MAX_TEAM and team * vpt < nvec:
        team *= 2
    while team * vpt < nvec:
        vpt *= 2
    while vpt > 1 and team * (vpt // 2) >= nvec:   # short rows: no idle vectors
        vpt //= 2
    teams = max(1, 128 // team)
    min_ctas = max(1, 1024 // (team * teams))
    row_bytes = rnumel * config.byte_per_numel(dtype) if dtype in config.BYTES_PER_ELEMENT else rnumel * 4
    streamed = rows is None or rows * row_bytes >= (64 << 20)
    return RowConfig(team=team, teams=teams, vpt=vpt, vec=vec, min_ctas=min_ctas,
                     prefetch=2 if streamed and row_bytes >= 2048 else 0)


def choose_loop_config(dtype: torch.dtype) -> RowConfig:
    """Launch shape of a row kernel that walks its rows in chunks: one team of 512 threads
    per CTA, two vectors per thread and chunk, registers bounded for two resident CTAs."""
    vec = min(max(config.get_aligned_numel(dtype), 1), 8)
    return RowConfig(team=512, teams=1, vpt=2, vec=vec, min_ctas=2, prefetch=0)


def row_candidates(rnumel: int, chosen: RowConfig, rows: Optional[int] = None, n_consts: int = 0,
                   kregs: int = 0):
    """Launch shapes worth measuring for a generated row kernel besides the chosen one:
    ``(team, teams, vpt, min_ctas, prefetch, kregs)`` tuples.  One, two and four vectors per
    thread over the matching power-of-two team; one, two or three teams per CTA; registers
    bounded for 256 to 1024 resident threads per SM; and, where the body has per-column
    operands, how many of them stay in registers (``kregs``; the rest are read from the
    shared-memory table, which frees registers for more resident warps).  The module loader
    builds the first few and keeps the one with the highest measured bandwidth
    (``codegen/jit.py``)."""
    vec = chosen.vec
    nvec = -(-rnumel // vec)
    default = (chosen.team, chosen.teams, chosen.vpt, chosen.min_ctas, chosen.prefetch, kregs)
    if chosen.team < 32:
        # rows of a few vectors: fewer lanes per row with more vectors each (shorter shuffle
        # trees, less index arithmetic per byte) against fully coalesced single vectors
        out = []
        for vpt in (2, 4):
            team = nvec // vpt
            if team < 2 or team * vpt != nvec or team & (team - 1):
                continue
            shape = (team, 128 // team, vpt, chosen.min_ctas, chosen.prefetch, kregs)
            if shape != default:
                out.append(shape)
        return out
    ranked = []
    for vpt in (1, 2, 4):
        team = 32
        while team < MAX_TEAM and team * vpt < nvec:
            team *= 2
        if team * vpt < nvec or (vpt > 1 and team * (vpt // 2) >= nvec):
            continue                      # does not cover the row / leaves idle vectors
        for teams in sorted({max(1, 128 // team), max(1, 256 // team), max(1, 384 // team)}):
            threads = team * teams
            if threads > 1024:
                continue
            for min_ctas in (1, 2, 3, 4):
                if threads * min_ctas > 1024 or (min_ctas > 1 and threads * min_ctas < 256):
                    continue
                for kr in sorted({kregs, min(n_consts, 1), 0}, reverse=True):
                    if kr > n_consts:
                        continue
                    shape = (team, teams, vpt, min_ctas, chosen.prefetch, kr)
                    if shape == default or shape in [s for _, s in ranked]:
                        continue
                    # prior for the order of measurement (from sweeps of the softmax ->
                    # LayerNorm chain): shapes whose registers fit their bound, thick threads
                    # first (the team exchange is paid per thread), then more resident warps
                    regs_const = kr * vpt * vec
                    fits = regs_const + 3 * vpt * vec + 40 <= 65536 // (threads * min_ctas)
                    score = (not fits, -vpt, -(threads * min_ctas), -kr)
                    ranked.append((score, shape))
    ranked.sort(key=lambda t: t[0])
    return [s for _, s in ranked]


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
