"""Segment (per-group) statistics on tensors without python loops.

Parity target: ``verl/utils/groupwise.py`` (``as_torch_index``, ``group_mean_std``).
"""

from __future__ import annotations

import numpy as np
import torch

__all__ = ["as_torch_index", "group_mean_std"]


def as_torch_index(index, device=None) -> torch.Tensor:
    """Dense int64 group ids (0..G-1, first-appearance order) from strings / ints / arrays / tensors."""
    if isinstance(index, torch.Tensor) and index.dtype in (torch.int32, torch.int64):
        _, inv = torch.unique(index, return_inverse=True)
        return inv.to(device=device, dtype=torch.int64)
    seq = index.tolist() if isinstance(index, (np.ndarray, torch.Tensor)) else list(index)
    table: dict = {}
    ids = [table.setdefault(v, len(table)) for v in seq]
    return torch.tensor(ids, dtype=torch.int64, device=device)


def group_mean_std(scores: torch.Tensor, gidx: torch.Tensor, eps: float = 1e-6):
    """(mean_g, std_g, count_g) per group; unbiased std; singleton groups report mean 0, std 1."""
    G = int(gidx.max().item()) + 1 if gidx.numel() else 0
    cnt = torch.bincount(gidx, minlength=G).to(scores.dtype)
    tot = torch.zeros(G, dtype=scores.dtype, device=scores.device).index_add_(0, gidx, scores)
    mean = tot / cnt.clamp(min=1)
    dev = torch.zeros(G, dtype=scores.dtype, device=scores.device).index_add_(0, gidx, (scores - mean[gidx]) ** 2)
    std = torch.sqrt(dev / (cnt - 1).clamp(min=1))
    single = cnt <= 1
    return torch.where(single, torch.zeros_like(mean), mean), torch.where(single, torch.ones_like(std), std), cnt
