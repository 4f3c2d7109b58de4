"""Sequence-length balancing: equal-cost partitions of a batch across ranks / micro-batches.

Workload model and partitioning follow ``verl/utils/seqlen_balancing.py`` (``calculate_workload`` :27-46,
Karmarkar-Karp :49, ``get_seqlen_balanced_partitions`` :213, ``rearrange_micro_batches`` :348-468).
"""

from __future__ import annotations

import heapq
from typing import Sequence

import torch
import torch.distributed as dist

__all__ = ["calculate_workload", "karmarkar_karp", "greedy_partition", "get_seqlen_balanced_partitions",
           "log_seqlen_unbalance", "rearrange_micro_batches", "get_reverse_idx", "restore_dynamic_batch",
           "get_group_balanced_partitions", "ceildiv", "roundup_divisible"]


def ceildiv(a: int, b: int) -> int:
    return -(a // -b)


def roundup_divisible(a: int, b: int) -> int:
    return ((a + b - 1) // b) * b


def calculate_workload(seqlen_list) -> torch.Tensor:
    """Relative cost of a sequence: linear term of the dense layers plus quadratic attention (24576*s + s^2)."""
    s = torch.as_tensor(seqlen_list, dtype=torch.int64)
    return 24576 * s + s * s


def karmarkar_karp(seqlen_list: Sequence[int], k_partitions: int, equal_size: bool) -> list[list[int]]:
    """Largest differencing method for k-way number partitioning."""

    class State:
        __slots__ = ("sets", "sums")

        def __init__(self, items, k):
            self.sets = [[] for _ in range(k)]
            self.sums = [0] * k
            for j, (idx, val) in enumerate(items):
                self.sets[j].append(idx)
                self.sums[j] = val

        def spread(self):
            return max(self.sums) - min(self.sums)

        def merge(self, other):
            a = sorted(range(len(self.sums)), key=lambda i: self.sums[i])
            b = sorted(range(len(other.sums)), key=lambda i: -other.sums[i])
            sets, sums = [], []
            for i, j in zip(a, b):
                sets.append(self.sets[i] + other.sets[j])
                sums.append(self.sums[i] + other.sums[j])
            self.sets, self.sums = sets, sums

        def __lt__(self, other):
            return self.spread() > other.spread()

    order = sorted(range(len(seqlen_list)), key=lambda i: seqlen_list[i])
    heap: list[State] = []
    if equal_size:
        assert len(seqlen_list) % k_partitions == 0, f"{len(seqlen_list)} % {k_partitions} != 0"
        for s in range(0, len(order), k_partitions):
            grp = [(i, seqlen_list[i]) for i in order[s : s + k_partitions]]
            heapq.heappush(heap, State(grp, k_partitions))
    else:
        for i in order:
            heapq.heappush(heap, State([(i, seqlen_list[i])], k_partitions))
    while len(heap) > 1:
        a, b = heapq.heappop(heap), heapq.heappop(heap)
        a.merge(b)
        heapq.heappush(heap, a)
    parts = heap[0].sets if heap else [[] for _ in range(k_partitions)]
    if equal_size:
        for p in parts:
            assert len(p) * k_partitions == len(seqlen_list)
    return parts


def greedy_partition(seqlen_list: Sequence[int], k_partitions: int, equal_size: bool) -> list[list[int]]:
    bias = sum(seqlen_list) + 1 if equal_size else 0
    parts = [[] for _ in range(k_partitions)]
    sums = [0] * k_partitions
    for i in sorted(range(len(seqlen_list)), key=lambda i: -seqlen_list[i]):
        j = min(range(k_partitions), key=lambda j: sums[j])
        parts[j].append(i)
        sums[j] += seqlen_list[i] + bias
    return parts


def get_seqlen_balanced_partitions(seqlen_list: Sequence[int], k_partitions: int, equal_size: bool) -> list[list[int]]:
    assert len(seqlen_list) >= k_partitions, f"number of items:[{len(seqlen_list)}] < k_partitions:[{k_partitions}]"
    parts = karmarkar_karp(list(seqlen_list), k_partitions, equal_size)
    seen = set()
    out = []
    for p in parts:
        assert len(p) > 0 or not equal_size
        seen.update(p)
        out.append(sorted(p))
    assert seen == set(range(len(seqlen_list)))
    return out


def log_seqlen_unbalance(seqlen_list: Sequence[int], partitions: list[list[int]], prefix: str) -> dict:
    k = len(partitions)
    bs = len(seqlen_list) // k
    naive = [sum(seqlen_list[i * bs : (i + 1) * bs]) for i in range(k)]
    bal = [sum(seqlen_list[i] for i in p) for p in partitions]
    return {f"{prefix}/min": min(naive), f"{prefix}/max": max(naive), f"{prefix}/minmax_diff": max(naive) - min(naive),
            f"{prefix}/balanced_min": min(bal), f"{prefix}/balanced_max": max(bal), f"{prefix}/mean": sum(naive) / k}


def get_reverse_idx(idx_map: Sequence[int]) -> list[int]:
    rev = [0] * len(idx_map)
    for i, j in enumerate(idx_map):
        rev[j] = i
    return rev


def rearrange_micro_batches(batch, max_token_len: int, dp_group=None, num_batches_divided_by=None, same_micro_num_in_dp=True,
                            min_num_micro_batch=None, use_dynamic_bsz_balance=True):
    """Split a batch (dict-like with ``attention_mask``) into micro-batches of at most ``max_token_len`` tokens.
    Returns (micro_batches, index_lists). The number of micro-batches is equalised across ``dp_group``."""
    mask = batch["attention_mask"]
    lens = mask.sum(dim=1)
    n = lens.shape[0]
    assert max_token_len >= int(lens.max()), f"max_token_len must be >= the longest sequence ({int(lens.max())})"
    k = min(n, ceildiv(int(lens.sum()), max_token_len))
    if min_num_micro_batch is not None:
        k = max(k, min_num_micro_batch)
    if dist.is_initialized() and same_micro_num_in_dp:
        t = torch.tensor([k], device=mask.device if mask.is_cuda else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=dp_group)
        k = int(t.item())
    if num_batches_divided_by is not None:
        k = roundup_divisible(k, num_batches_divided_by)
    k = min(k, n)
    parts = get_seqlen_balanced_partitions(lens.tolist(), k, equal_size=False)
    if use_dynamic_bsz_balance:
        parts.sort(key=lambda p: (-sum(int(calculate_workload([lens[i]])) for i in p), p[0] if p else 0))
    mbs = []
    for p in parts:
        idx = torch.tensor(p, dtype=torch.int64)
        mbs.append({k_: (v[idx.to(v.device)] if isinstance(v, torch.Tensor) and v.dim() > 0 and v.shape[0] == n else v)
                    for k_, v in batch.items()})
    return mbs, parts


def restore_dynamic_batch(data: torch.Tensor, batch_idx_list: list[list[int]]) -> torch.Tensor:
    flat = sum(batch_idx_list, [])
    rev = torch.tensor(get_reverse_idx(flat), dtype=torch.long, device=data.device)
    return data[rev]


def get_group_balanced_partitions(seqlen_list: Sequence[int], group_ids: Sequence, k_partitions: int) -> list[list[int]]:
    """Balance whole groups (all samples of one prompt stay together) across ``k_partitions``."""
    groups: dict = {}
    for i, g in enumerate(group_ids):
        groups.setdefault(g, []).append(i)
    keys = list(groups)
    costs = [int(sum(int(calculate_workload([seqlen_list[i]])) for i in groups[g])) for g in keys]
    parts = get_seqlen_balanced_partitions(costs, k_partitions, equal_size=len(keys) % k_partitions == 0)
    return [sorted(i for gi in p for i in groups[keys[gi]]) for p in parts]
