"""Dynamic context parallelism: a context-parallel group size per sample instead of one for the whole run.

A block of ``cp_size`` ranks holds the same rows. With a fixed group size every row is cut over all ``cp_size`` ranks,
which wastes communication on the short rows of a batch whose longest row needs the whole block. Here every row gets the
smallest power-of-two group that keeps ``ceil(length / group) <= max_seqlen_per_dp_cp_rank``; groups are aligned windows
of the block's ranks (size s starts at a multiple of s), so one process group per (size, window) serves every step. The
scheduler packs the rows into micro-batches: inside one micro-batch a rank belongs to exactly one group (it runs one
forward / backward with one communication pattern), several rows may share a group while its ranks have room, and rows are
placed longest-group-first into the window with the lightest load, which balances the ranks.

Parity target: ``verl/utils/dynamic_cp_scheduler.py`` (``DynamicCPScheduler.schedule`` :127-210, a thin adapter over
Megatron-Core's ``DefaultDynamicCPScheduler``; the packing itself is this module's own) and
``verl/workers/config/engine.py`` (``dynamic_context_parallel``, ``max_seqlen_per_dp_cp_rank``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

__all__ = ["DynamicCPScheduler", "GroupAssignment", "required_group_size"]


def required_group_size(seq_len: int, max_seqlen_per_rank: int, cp_size: int) -> int:
    """Smallest power of two s with ceil(seq_len / s) <= max_seqlen_per_rank; raises when even the whole block is too small."""
    need = max(1, math.ceil(seq_len / max_seqlen_per_rank))
    s = 1
    while s < need:
        s *= 2
    if s > cp_size:
        raise ValueError(f"A sequence with {seq_len} tokens needs at least {need} ranks at max_seqlen_per_dp_cp_rank="
                         f"{max_seqlen_per_rank}, but the context-parallel block only has {cp_size} ranks. Increase "
                         f"max_seqlen_per_dp_cp_rank or cap the sequence length.")
    return s


@dataclass
class GroupAssignment:
    """What one rank does in one micro-batch: the rows it works on with the ranks ``[start, start + size)`` of its block."""

    size: int = 1
    start: int = 0
    rows: list = field(default_factory=list)


class _MicroBatch:
    def __init__(self, cp_size: int):
        self.load = [0.0] * cp_size                 # tokens per rank
        self.width: list[Optional[int]] = [None] * cp_size   # group size a rank is committed to in this micro-batch
        self.groups: dict[tuple[int, int], list[int]] = {}   # (size, start) -> rows

    def best_window(self, s: int, per_rank: float, cap: float) -> Optional[int]:
        best, best_load = None, None
        for w in range(0, len(self.load), s):
            ranks = range(w, w + s)
            if any(self.width[r] not in (None, s) for r in ranks):
                continue
            if any(self.width[r] == s for r in ranks) and (s, w) not in self.groups:
                continue  # committed to a group of this size in another window (cannot happen with aligned windows; kept as a guard)
            top = max(self.load[r] for r in ranks)
            if top + per_rank > cap and top > 0:
                continue
            if best is None or top < best_load:
                best, best_load = w, top
        return best

    def place(self, row: int, s: int, w: int, per_rank: float) -> None:
        for r in range(w, w + s):
            self.load[r] += per_rank
            self.width[r] = s
        self.groups.setdefault((s, w), []).append(row)


class DynamicCPScheduler:
    def __init__(self, max_seqlen_per_dp_cp_rank: int, cp_size: int):
        if any(type(v) is not int or v <= 0 for v in (max_seqlen_per_dp_cp_rank, cp_size)):
            raise ValueError("Dynamic CP scheduler sizes must be positive integers")
        if cp_size & (cp_size - 1):
            raise ValueError(f"the context-parallel block size must be a power of two, got {cp_size}")
        self.max_seqlen, self.cp_size = max_seqlen_per_dp_cp_rank, cp_size

    def schedule(self, seq_lens: list[int]) -> list[list[GroupAssignment]]:
        """Micro-batches for rows of the given lengths: ``result[m][r]`` is what rank ``r`` of the block does in micro-batch
        ``m`` (``rows`` empty: the rank sits this one out). Every row appears in exactly one group of one micro-batch, with
        the same row list (same order) on every rank of that group."""
        if not seq_lens:
            raise ValueError("Dynamic CP cannot schedule an empty batch")
        if any(int(n) <= 0 for n in seq_lens):
            raise ValueError("Dynamic CP requires every input sequence to contain at least one token")
        sizes = [required_group_size(int(n), self.max_seqlen, self.cp_size) for n in seq_lens]
        order = sorted(range(len(seq_lens)), key=lambda i: (-sizes[i], -int(seq_lens[i]), i))
        mbs: list[_MicroBatch] = []
        for i in order:
            s, per_rank = sizes[i], int(seq_lens[i]) / sizes[i]
            for mb in mbs:
                w = mb.best_window(s, per_rank, self.max_seqlen)
                if w is not None:
                    mb.place(i, s, w, per_rank)
                    break
            else:
                mb = _MicroBatch(self.cp_size)
                mb.place(i, s, mb.best_window(s, per_rank, self.max_seqlen), per_rank)
                mbs.append(mb)
        out = []
        for mb in mbs:
            ranks = [GroupAssignment() for _ in range(self.cp_size)]
            for (s, w), rows in mb.groups.items():
                for r in range(w, w + s):
                    ranks[r] = GroupAssignment(size=s, start=w, rows=sorted(rows))
            out.append(ranks)
        return out

    def loads(self, seq_lens: list[int], plan: list[list[GroupAssignment]]) -> list[list[float]]:
        """Tokens per rank and micro-batch of a plan (diagnostics and tests)."""
        return [[sum(seq_lens[i] / a.size for i in a.rows) for a in mb] for mb in plan]
