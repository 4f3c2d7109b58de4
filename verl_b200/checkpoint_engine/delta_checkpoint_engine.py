"""Sparse delta synchronisation: only elements whose bf16 bit pattern changed since the last synchronised
snapshot travel, as (index, value) pairs, with a checksum to detect drift.

Parity target: ``verl/checkpoint_engine/delta_checkpoint_engine.py`` (672 lines) and ``delta_sync/{encode,
sparse_gather}.py``.
"""

from __future__ import annotations

from typing import Iterable, Optional

import torch
import torch.distributed as dist

from .base import CheckpointEngine, CheckpointEngineRegistry

__all__ = ["encode_delta", "apply_delta", "tensor_checksum", "sparse_gather", "DeltaCheckpointEngine"]


def _bits(t: torch.Tensor) -> torch.Tensor:
    v = t.detach().contiguous().view(-1)
    return v.view({2: torch.int16, 4: torch.int32, 1: torch.int8, 8: torch.int64}[v.element_size()])


def encode_delta(new: torch.Tensor, snapshot: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(indices int64, values) of the elements of ``new`` whose bits differ from ``snapshot``."""
    idx = torch.nonzero(_bits(new) != _bits(snapshot), as_tuple=False).view(-1)
    return idx, new.detach().contiguous().view(-1)[idx]


def apply_delta(target: torch.Tensor, idx: torch.Tensor, values: torch.Tensor) -> None:
    target.view(-1)[idx.to(target.device)] = values.to(device=target.device, dtype=target.dtype)


def tensor_checksum(t: torch.Tensor) -> int:
    """Order-independent 64-bit sum of the raw bits (cheap drift detector)."""
    return int(_bits(t).to(torch.int64).sum().item())


def sparse_gather(idx: torch.Tensor, val: torch.Tensor, dst: int = 0, group=None):
    """Gather variable-length (idx, val) pairs on ``dst``: all-gather the counts, pad to the maximum, gather."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n = torch.tensor([idx.numel()], dtype=torch.int64, device=idx.device)
    counts = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(counts, n, group=group)
    counts = [int(c) for c in counts]
    mx = max(counts) if counts else 0
    pi = torch.zeros(mx, dtype=idx.dtype, device=idx.device)
    pv = torch.zeros(mx, dtype=val.dtype, device=val.device)
    pi[: idx.numel()], pv[: val.numel()] = idx, val
    gi = [torch.zeros_like(pi) for _ in range(world)] if rank == dst else None
    gv = [torch.zeros_like(pv) for _ in range(world)] if rank == dst else None
    dist.gather(pi, gi, dst=dst, group=group)
    dist.gather(pv, gv, dst=dst, group=group)
    if rank != dst:
        return None
    return [(gi[r][: counts[r]], gv[r][: counts[r]]) for r in range(world)]


@CheckpointEngineRegistry.register("delta_sharded")
class DeltaCheckpointEngine(CheckpointEngine):
    """Sender keeps a snapshot per tensor; the first sync ships everything, later syncs ship deltas. The receiver
    applies them onto its resident weights and verifies the checksum."""

    def __init__(self, group=None, src: int = 0, device=None, full_sync_every: int = 0, **kwargs):
        self.group, self.src, self.device = group, src, device
        self.snapshots: dict[str, torch.Tensor] = {}
        self.resident: dict[str, torch.Tensor] = {}
        self.full_sync_every = full_sync_every
        self.num_syncs = 0
        self.last_stats: dict = {}

    def prepare(self):
        return None

    @classmethod
    def build_topology(cls, trainer_world_size, rollout_world_size, metadata):
        world = 1 + rollout_world_size
        return ({"rank": [0] + [-1] * (trainer_world_size - 1)}, {"rank": list(range(1, world))})

    def init_process_group(self, group=None, src: int = 0, **kwargs):
        if group is not None:
            self.group, self.src = group, src

    def finalize(self):
        return None

    def _bcast_obj(self, obj=None):
        box = [obj]
        dist.broadcast_object_list(box, src=self.src, group=self.group)
        return box[0]

    async def send_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> None:
        full = self.num_syncs == 0 or (self.full_sync_every and self.num_syncs % self.full_sync_every == 0)
        sent = total = 0
        for name, t in weights:
            flat = t.detach().contiguous().view(-1)
            total += flat.numel()
            if full or name not in self.snapshots:
                idx = torch.arange(flat.numel(), device=flat.device)
                val = flat
            else:
                idx, val = encode_delta(flat, self.snapshots[name])
            self.snapshots[name] = flat.clone()
            sent += idx.numel()
            hdr = {"name": name, "shape": tuple(t.shape), "dtype": t.dtype, "n": int(idx.numel()), "full": bool(full),
                   "checksum": tensor_checksum(flat)}
            self._bcast_obj(hdr)
            if idx.numel():
                dist.broadcast(idx.to(torch.int64), src=self.src, group=self.group)
                dist.broadcast(val.contiguous(), src=self.src, group=self.group)
        self._bcast_obj(None)
        self.num_syncs += 1
        self.last_stats = {"sent_elements": sent, "total_elements": total, "density": sent / max(1, total)}

    async def receive_weights(self):
        while True:
            hdr = self._bcast_obj()
            if hdr is None:
                break
            name, n = hdr["name"], hdr["n"]
            if name not in self.resident:
                self.resident[name] = torch.zeros(hdr["shape"], dtype=hdr["dtype"], device=self.device or "cpu")
            tgt = self.resident[name]
            if n:
                idx = torch.empty(n, dtype=torch.int64, device=tgt.device)
                val = torch.empty(n, dtype=hdr["dtype"], device=tgt.device)
                dist.broadcast(idx, src=self.src, group=self.group)
                dist.broadcast(val, src=self.src, group=self.group)
                apply_delta(tgt, idx, val)
            if tensor_checksum(tgt) != hdr["checksum"]:
                raise RuntimeError(f"delta sync checksum mismatch on '{name}': receiver state drifted; request a full sync")
            yield name, tgt
