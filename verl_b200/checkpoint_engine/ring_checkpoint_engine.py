"""Pipelined relay of weight buckets along a chain of ranks: the trainer's sender passes bucket k to the first rollout
rank, which forwards it to the next one while it already receives bucket k + 1, and so on. Every link carries each
byte once, so the sender's egress does not grow with the number of receivers (a broadcast from one rank does), and with
B buckets over R receivers the transfer takes about (B + R - 1) bucket times.

This is the topology of the reference's RDMA transports; here the links are ``torch.distributed`` point-to-point
messages (NCCL over NVLink on GPUs, gloo on CPU), which is why the same engine is registered under the names of those
transports: ``nixl`` and ``mooncake`` (ring of trainer and rollout ranks), ``kimi`` (point-to-point hand-off followed by
relays) and ``hccl``.

Parity target: ``verl/checkpoint_engine/nixl_checkpoint_engine.py`` (ring of agents, double-buffered buckets),
``mooncake_checkpoint_engine.py``, ``kimi_checkpoint_engine.py``, ``hccl_checkpoint_engine.py``.
"""

from __future__ import annotations

from typing import Any, Iterable, Optional

import torch
import torch.distributed as dist

from .base import CheckpointEngine, CheckpointEngineRegistry, TensorMeta, _ChunkAssembler, bucketize

__all__ = ["RingCheckpointEngine"]


@CheckpointEngineRegistry.register("ring")
@CheckpointEngineRegistry.register("nixl")
@CheckpointEngineRegistry.register("mooncake")
@CheckpointEngineRegistry.register("kimi")
@CheckpointEngineRegistry.register("hccl")
class RingCheckpointEngine(CheckpointEngine):
    def __init__(self, bucket_size: int = 512 << 20, group=None, src: int = 0, device=None, is_master: bool = False, **kwargs):
        self.bucket_size = int(bucket_size)
        self.group, self.src, self.device, self.is_master = group, src, device, is_master

    def prepare(self) -> Any:
        return {"bucket_size": self.bucket_size}

    @classmethod
    def build_topology(cls, trainer_world_size: int, rollout_world_size: int, metadata: list):
        world = 1 + rollout_world_size  # chain: trainer rank 0 -> rollout 0 -> rollout 1 -> ...
        trainer = {"rank": [0] + [-1] * (trainer_world_size - 1), "world_size": [world] * trainer_world_size}
        rollout = {"rank": list(range(1, world)), "world_size": [world] * rollout_world_size}
        return trainer, rollout

    def init_process_group(self, group=None, src: int = 0, **kwargs) -> None:
        if group is not None:
            self.group, self.src = group, src

    def finalize(self) -> None:
        return None

    # ---- chain positions (ranks of the group, starting at the sender)
    def _chain(self) -> tuple[int, int, Optional[int], Optional[int]]:
        world, me = dist.get_world_size(self.group), dist.get_rank(self.group)
        pos = (me - self.src) % world
        g = (lambda r: dist.get_global_rank(self.group, r)) if self.group is not None else (lambda r: r)
        prev = g((me - 1) % world) if pos > 0 else None
        nxt = g((me + 1) % world) if pos < world - 1 else None
        return world, pos, prev, nxt

    def _send_obj(self, obj, dst: int) -> None:
        dist.send_object_list([obj], dst=dst, group=self.group)

    def _recv_obj(self, src: int):
        box = [None]
        dist.recv_object_list(box, src=src, group=self.group)
        return box[0]

    async def send_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> None:
        _, _, _, nxt = self._chain()
        if nxt is None:
            return
        pending = None
        for bucket, metas in bucketize(weights, self.bucket_size, device=self.device):
            self._send_obj(metas, nxt)
            if pending is not None:
                pending[0].wait()  # at most two buckets alive: the one in flight and the one being packed
            pending = (dist.isend(bucket, dst=nxt, group=self.group), bucket)
        if pending is not None:
            pending[0].wait()
        self._send_obj(None, nxt)  # end of stream

    async def receive_weights(self):
        _, _, prev, nxt = self._chain()
        asm = _ChunkAssembler()
        bufs = [torch.empty(self.bucket_size, dtype=torch.uint8, device=self.device or "cpu") for _ in range(2)]
        fwd = [None, None]  # forward of the bucket that used buffer i
        k = 0
        while True:
            metas: Optional[list[TensorMeta]] = self._recv_obj(prev)
            if nxt is not None:
                self._send_obj(metas, nxt)
            if metas is None:
                break
            i = k & 1
            if fwd[i] is not None:
                fwd[i].wait()  # the buffer is still being forwarded from two buckets ago
                fwd[i] = None
            dist.recv(bufs[i], src=prev, group=self.group)
            if nxt is not None:
                fwd[i] = dist.isend(bufs[i], dst=nxt, group=self.group)  # relay while the tensors are unpacked below
            for name, t in asm.feed(bufs[i], metas):
                yield name, t
            k += 1
        for w in fwd:
            if w is not None:
                w.wait()
