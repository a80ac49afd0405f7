"""Partitioning of decode work over several GPUs.

The decode path has no exchange step: every output texel depends only on the (small, read-only)
compressed set.  Work is therefore split by texture set, by mip and by tile rows, each GPU holds
a full copy of the compressed sets it touches, and nothing but the final host gather crosses
between ranks.  (The reference has no multi-GPU code; one `ntc::Context` drives one device,
include/libntc/ntc.h:1289-1290.)

Two plans:
  * `plan_batch`   many independent sets (e.g. 64 sets of 2048^2): units are (set, mip 0) and
                   (set, mips >= 1) - mip 0 is 75 % of a set - assigned longest-first to the least
                   loaded rank;
  * `plan_rows`    one large set: every mip tall enough is cut into one band of tile rows per rank,
                   the small mips go whole, largest first, to the least loaded rank.
Row bands are multiples of the kernel's tile height so that no tile straddles two ranks.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

from .geometry import Geometry

TILE_ROWS = 8          # the decode kernel's tile height
MIN_ROWS_PER_RANK = 64  # mips shorter than world * this are not split


@dataclass(frozen=True)
class WorkUnit:
    set_index: int
    mips: Tuple[int, ...]
    texels: int


def plan_batch(geometries: Sequence[Geometry], world: int) -> List[List[WorkUnit]]:
    """Longest-processing-time-first assignment of (set, mip group) units to `world` ranks."""
    if world < 1:
        raise ValueError("world must be positive")
    units: List[WorkUnit] = []
    for index, geo in enumerate(geometries):
        first = geo.color_mips[0]
        units.append(WorkUnit(index, (0,), first.width * first.height))
        if geo.mips > 1:
            rest = sum(cm.width * cm.height for cm in geo.color_mips[1:])
            units.append(WorkUnit(index, tuple(range(1, geo.mips)), rest))
    units.sort(key=lambda u: (-u.texels, u.set_index, u.mips))
    plan: List[List[WorkUnit]] = [[] for _ in range(world)]
    load = [0] * world
    for unit in units:
        rank = min(range(world), key=lambda r: (load[r], r))
        plan[rank].append(unit)
        load[rank] += unit.texels
    return plan


def plan_rows(geo: Geometry, world: int) -> List[List[Tuple[int, int]]]:
    """Row range [begin, end) of every mip for every rank: plan[rank][mip]."""
    if world < 1:
        raise ValueError("world must be positive")
    plan = [[(0, 0)] * geo.mips for _ in range(world)]
    load = [0] * world
    whole = []
    for mip, cm in enumerate(geo.color_mips):
        if cm.height < world * MIN_ROWS_PER_RANK:
            whole.append(mip)
            continue
        tiles = (cm.height + TILE_ROWS - 1) // TILE_ROWS
        for rank in range(world):
            begin = (tiles * rank // world) * TILE_ROWS
            end = min(cm.height, (tiles * (rank + 1) // world) * TILE_ROWS)
            plan[rank][mip] = (begin, end)
            load[rank] += (end - begin) * cm.width
    # the mips too short to split go whole, largest first, to the rank with the least work so far
    for mip in sorted(whole, key=lambda m: -geo.color_mips[m].width * geo.color_mips[m].height):
        cm = geo.color_mips[mip]
        rank = min(range(world), key=lambda r: (load[r], r))
        plan[rank][mip] = (0, cm.height)
        load[rank] += cm.width * cm.height
    return plan


def texels_of_rows(geo: Geometry, ranges: Sequence[Tuple[int, int]]) -> int:
    return sum((end - begin) * geo.color_mips[mip].width for mip, (begin, end) in enumerate(ranges))


def unit_row_ranges(geo: Geometry, unit: WorkUnit) -> List[Tuple[int, int]]:
    """Per-mip row ranges that decode exactly the mips of `unit`."""
    return [(0, cm.height) if mip in unit.mips else (0, 0) for mip, cm in enumerate(geo.color_mips)]
