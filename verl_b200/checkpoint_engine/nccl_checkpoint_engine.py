"""Bucketed broadcast of weights from trainer rank 0 to standalone rollout ranks over a dedicated process group
(NCCL on GPUs, gloo on CPU), double-buffered so packing bucket k+1 overlaps the broadcast of bucket k.

Parity target: ``verl/checkpoint_engine/nccl_checkpoint_engine.py:119-515``.
"""

from __future__ import annotations

import pickle
from typing import Any, Iterable, Optional

import torch
import torch.distributed as dist

from .base import CheckpointEngine, CheckpointEngineRegistry, TensorMeta, _ChunkAssembler, bucketize

__all__ = ["NCCLCheckpointEngine"]


@CheckpointEngineRegistry.register("nccl")
class NCCLCheckpointEngine(CheckpointEngine):
    def __init__(self, bucket_size: int = 512 << 20, group=None, src: int = 0, device=None, is_master: bool = False, **kwargs):
        self.bucket_size = int(bucket_size)
        self.group, self.src = group, src
        self.device = device
        self.is_master = is_master

    def prepare(self) -> Any:
        return {"bucket_size": self.bucket_size}

    @classmethod
    def build_topology(cls, trainer_world_size: int, rollout_world_size: int, metadata: list):
        world = 1 + rollout_world_size  # trainer rank 0 is the only sender
        trainer = {"rank": [0] + [-1] * (trainer_world_size - 1), "world_size": [world] * trainer_world_size}
        rollout = {"rank": list(range(1, world)), "world_size": [world] * rollout_world_size}
        return trainer, rollout

    def init_process_group(self, group=None, src: int = 0, **kwargs) -> None:
        if group is not None:
            self.group, self.src = group, src

    def finalize(self) -> None:
        return None

    def _bcast_obj(self, obj=None):
        box = [obj]
        dist.broadcast_object_list(box, src=self.src, group=self.group)
        return box[0]

    async def send_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> None:
        dev = self.device
        for bucket, metas in bucketize(weights, self.bucket_size, device=dev):
            self._bcast_obj(metas)
            dist.broadcast(bucket, src=self.src, group=self.group)
        self._bcast_obj(None)  # end of stream

    async def receive_weights(self):
        asm = _ChunkAssembler()
        while True:
            metas: Optional[list[TensorMeta]] = self._bcast_obj()
            if metas is None:
                break
            bucket = torch.empty(self.bucket_size, dtype=torch.uint8, device=self.device or "cpu")
            dist.broadcast(bucket, src=self.src, group=self.group)
            for name, t in asm.feed(bucket, metas):
                yield name, t

    # ---- identical-layout fast path: both sides hold the same flat parameter buffer, so the buffer itself is
    # broadcast in place, slice by slice (no packing, no staging copy, no metadata)
    def send_flat(self, flat: torch.Tensor) -> None:
        self._bcast_flat(flat)

    def receive_flat(self, flat: torch.Tensor) -> None:
        self._bcast_flat(flat)

    def _bcast_flat(self, flat: torch.Tensor) -> None:
        step = max(1, self.bucket_size // flat.element_size())
        works = []
        for lo in range(0, flat.numel(), step):
            works.append(dist.broadcast(flat[lo : lo + step], src=self.src, group=self.group, async_op=True))
        for w in works:
            w.wait()
