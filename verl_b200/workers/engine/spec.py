"""Shard-export contract between a training engine and the sharded weight-sync back-ends.

``engine.get_per_tensor_param_shard()`` yields ``(name, local_shard, ShardSpec)`` in an order identical on all ranks. The
native engine shards ONE flat buffer contiguously over the data-parallel ranks, so a tensor's local shard is the
intersection of the tensor's flat range with this rank's slice: ``ShardSpec.place`` is the flat offset of that piece
inside the full tensor and ``gather_group`` the data-parallel group. ``translate_flat_indices`` maps indices of changed
elements in the local piece to indices in the full tensor (what a sparse delta ships).

Parity target: ``verl/workers/engine/spec.py`` (``ShardSpec``, ``BlockPlacement``, ``translate_flat_indices``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch

__all__ = ["BlockPlacement", "ShardSpec", "translate_flat_indices", "flat_range_shards"]


@dataclass
class BlockPlacement:
    """A rectangular block of a (virtual) full tensor: per-dimension start offsets and the block's shape."""

    starts: tuple
    shape: tuple


@dataclass
class ShardSpec:
    full_shape: tuple
    place: Optional[int | BlockPlacement] = None  # flat offset or block of the local shard inside the full tensor; None = whole
    gather_group: Any = None                       # group of the ranks that together hold the tensor; None = unsharded
    contributes: bool = True                       # False: this rank's piece is a replica owned by a peer

    @property
    def numel(self) -> int:
        n = 1
        for d in self.full_shape:
            n *= int(d)
        return n


def translate_flat_indices(local_idx: torch.Tensor, spec: ShardSpec) -> torch.Tensor:
    """Indices into the flattened local shard -> indices into the flattened full tensor."""
    if spec.place is None:
        return local_idx
    if isinstance(spec.place, int):
        return local_idx + spec.place
    bp = spec.place
    strides_full, s = [], 1
    for d in reversed(spec.full_shape):
        strides_full.append(s)
        s *= int(d)
    strides_full = list(reversed(strides_full))
    out = torch.zeros_like(local_idx)
    rem = local_idx.clone()
    inner = 1
    dims = list(bp.shape)
    for i in reversed(range(len(dims))):
        coord = (rem // inner) % dims[i] if i > 0 else rem // inner
        out += (coord + bp.starts[i]) * strides_full[i]
        inner *= dims[i]
    return out


def flat_range_shards(params, shard_lo: int, shard_numel: int, group=None):
    """(name, local piece, ShardSpec) for every tensor of a flat parameter buffer that intersects the flat range
    ``[shard_lo, shard_lo + shard_numel)`` owned by this rank."""
    hi = shard_lo + shard_numel
    for name, view in params.views.items():
        off = params.offsets[name][0] if isinstance(params.offsets[name], (tuple, list)) else int(params.offsets[name])
        n = view.numel()
        a, b = max(off, shard_lo), min(off + n, hi)
        if a >= b:
            yield name, view.reshape(-1)[:0], ShardSpec(tuple(view.shape), place=0, gather_group=group, contributes=False)
            continue
        yield name, params.flat[a:b], ShardSpec(tuple(view.shape), place=a - off, gather_group=group, contributes=True)
