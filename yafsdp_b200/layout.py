"""Closed-form ragged flat layout of one parameter group.

All parameters of a group are laid end to end (row-major flattening, no per-parameter padding) in
one flat vector that is padded to ``world_size * shard_alignment`` elements and cut into
``world_size`` equal contiguous shards, irrespective of parameter boundaries.  A parameter may span
several ranks and a rank may own nothing of a parameter.  Everything is computed with integer
arithmetic on the host in O(#params * world): no index tensors, no device work, no ``.item()``.

Parity: the reference derives the same quantities with per-element index tensors
(``ya_fsdp/_param_group.py:241-377``); the resulting numbers are identical (see the layout tests).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence


def round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass(frozen=True)
class ParamPlacement:
    """Where one parameter lives in the flat vector and in one rank's shard."""

    index: int
    numel: int
    flat_offset: int  # start of the parameter in the unsharded flat vector
    local_numel: int  # elements of the parameter owned by the rank
    global_offset: int  # offset inside the flattened parameter of the first owned element (== numel if none)
    shard_offset: int  # offset inside the rank's shard of the first owned element
    shard_numels: tuple[int, ...]  # owned elements per rank


class FlatLayout:
    """Flat ragged layout of ``numels`` over ``world_size`` ranks."""

    def __init__(self, numels: Sequence[int], world_size: int, shard_alignment: int = 8):
        if world_size < 1:
            raise ValueError("world_size must be >= 1")
        if shard_alignment < 1:
            raise ValueError("shard_alignment must be >= 1")
        self.numels = tuple(int(n) for n in numels)
        self.world_size = world_size
        self.shard_alignment = shard_alignment
        offs = []
        o = 0
        for n in self.numels:
            offs.append(o)
            o += n
        self.flat_offsets = tuple(offs)
        self.total_numel = o
        self.padded_numel = round_up(max(o, 1), world_size * shard_alignment)
        self.shard_numel = self.padded_numel // world_size

    def shard_range(self, rank: int) -> tuple[int, int]:
        return rank * self.shard_numel, (rank + 1) * self.shard_numel

    def _overlap(self, index: int, rank: int) -> tuple[int, int]:
        o, n = self.flat_offsets[index], self.numels[index]
        lo_r, hi_r = self.shard_range(rank)
        lo, hi = max(o, lo_r), min(o + n, hi_r)
        return (lo, hi) if hi > lo else (o + n, o + n)

    def shard_numels(self, index: int) -> tuple[int, ...]:
        out = []
        for r in range(self.world_size):
            lo, hi = self._overlap(index, r)
            out.append(hi - lo)
        return tuple(out)

    def placement(self, index: int, rank: int) -> ParamPlacement:
        o, n = self.flat_offsets[index], self.numels[index]
        lo, hi = self._overlap(index, rank)
        local = hi - lo
        lo_r, _ = self.shard_range(rank)
        return ParamPlacement(
            index=index,
            numel=n,
            flat_offset=o,
            local_numel=local,
            global_offset=(lo - o) if local > 0 else n,
            shard_offset=(lo - lo_r) if local > 0 else min(max(o - lo_r, 0), self.shard_numel),
            shard_numels=self.shard_numels(index),
        )

    def placements(self, rank: int) -> list[ParamPlacement]:
        return [self.placement(i, rank) for i in range(len(self.numels))]

    def owners(self, index: int) -> list[int]:
        """Ranks that own at least one element of the parameter."""
        return [r for r, n in enumerate(self.shard_numels(index)) if n > 0]

    def __repr__(self) -> str:
        return (
            f"FlatLayout(params={len(self.numels)}, total={self.total_numel}, padded={self.padded_numel}, "
            f"world={self.world_size}, shard={self.shard_numel})"
        )


def reshard_ranges(numel: int, old_shard_numels: Sequence[int], new_lo: int, new_hi: int) -> list[tuple[int, int, int]]:
    """Pieces ``(old_rank, old_local_offset, length)`` of a flattened parameter (stored as ragged shards
    of ``old_shard_numels`` elements per old rank) that cover the flat range ``[new_lo, new_hi)``.
    Used when loading a checkpoint into a different world size."""
    out = []
    start = 0
    for r, n in enumerate(old_shard_numels):
        lo, hi = max(start, new_lo), min(start + n, new_hi)
        if hi > lo:
            out.append((r, lo - start, hi - lo))
        start += n
    assert start == numel or not old_shard_numels
    return out
