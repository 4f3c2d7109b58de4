"""Weight synchronisation between trainer and rollout replicas ("checkpoint engines").

``naive`` is the colocated case: trainer and rollout share the working weights, the engine only forwards the
(name, tensor) stream.  The other back-ends move weights to replicas that live on other GPUs: bucketed
broadcast over a process group (``nccl``) or sparse deltas against the last synchronised snapshot
(``delta_sharded``).

Parity target: ``verl/checkpoint_engine/base.py`` (``TensorMeta`` :33, registry :49, ``CheckpointEngine`` ABC
:116-225, ``ColocatedCheckpointEngine`` :245-300, ``CheckpointEngineManager`` :378-558, chunk helpers :561-629).
"""

from __future__ import annotations

import asyncio
import time
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, AsyncGenerator, Generator, Iterable, Optional

import torch

__all__ = ["TensorMeta", "CheckpointEngine", "CheckpointEngineRegistry", "ColocatedCheckpointEngine",
           "CheckpointEngineManager", "split_weight_chunks", "merge_weight_chunks", "bucketize"]


@dataclass
class TensorMeta:
    name: str
    shape: tuple
    dtype: torch.dtype
    offset: int  # byte offset inside the bucket
    nbytes: int = 0
    chunk_offset: Optional[int] = None  # for tensors split across buckets
    chunk_size: Optional[int] = None


class CheckpointEngineRegistry:
    _registry: dict[str, type["CheckpointEngine"]] = {}

    @classmethod
    def register(cls, backend: str):
        def deco(engine_cls):
            cls._registry[backend] = engine_cls
            return engine_cls

        return deco

    # transports of the reference whose libraries are absent here: they run the relay ring over torch.distributed p2p
    ALIASES = {"nixl": "ring", "mooncake": "ring", "kimi": "ring", "hccl": "ring"}
    _warned: set = set()

    @classmethod
    def get(cls, backend: str) -> type["CheckpointEngine"]:
        if backend in cls.ALIASES and backend not in cls._warned:
            import warnings

            cls._warned.add(backend)
            warnings.warn(f"checkpoint engine '{backend}' is served by the '{cls.ALIASES[backend]}' relay chain over torch.distributed "
                          f"point-to-point messages (the {backend} transport library is not part of this framework)", stacklevel=2)
        if backend not in cls._registry:
            from . import delta_checkpoint_engine, nccl_checkpoint_engine, ring_checkpoint_engine  # noqa: F401  (self-registering)
        if backend not in cls._registry:
            raise ValueError(f"Checkpoint engine {backend} not registered (known: {sorted(cls._registry)})")
        return cls._registry[backend]

    @classmethod
    def new(cls, backend: str, *args, **kwargs) -> "CheckpointEngine":
        return cls.get(backend)(*args, **kwargs)


class CheckpointEngine(ABC):
    """prepare -> build_topology -> init_process_group -> send_weights / receive_weights -> finalize."""

    @abstractmethod
    def prepare(self) -> Any:
        """Allocate transfer buffers; returns metadata to exchange (addresses, ports)."""

    @classmethod
    @abstractmethod
    def build_topology(cls, trainer_world_size: int, rollout_world_size: int, metadata: list) -> tuple[dict, dict]:
        """Per-rank keyword arguments of ``init_process_group`` for trainer ranks and rollout ranks."""

    @abstractmethod
    def init_process_group(self, **kwargs) -> None:
        ...

    @abstractmethod
    def finalize(self) -> None:
        ...

    @abstractmethod
    async def send_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> None:
        ...

    @abstractmethod
    async def receive_weights(self) -> AsyncGenerator[tuple[str, torch.Tensor], None]:
        ...


@CheckpointEngineRegistry.register("naive")
class ColocatedCheckpointEngine(CheckpointEngine):
    """Same-process hand-over: the generator of trainer tensors is what the rollout consumes."""

    def __init__(self, bucket_size: int = 0, is_master: bool = False, **kwargs):
        self.bucket_size, self.is_master = bucket_size, is_master
        self._weights: Optional[Iterable] = None

    def prepare(self):
        return None

    @classmethod
    def build_topology(cls, trainer_world_size, rollout_world_size, metadata):
        return {"rank": list(range(trainer_world_size))}, {"rank": list(range(rollout_world_size))}

    def init_process_group(self, **kwargs):
        return None

    def finalize(self):
        self._weights = None

    async def send_weights(self, weights):
        self._weights = weights

    async def receive_weights(self):
        for name, t in (self._weights or ()):
            yield name, t
        self._weights = None


def bucketize(weights: Iterable[tuple[str, torch.Tensor]], bucket_bytes: int, device=None
              ) -> Generator[tuple[torch.Tensor, list[TensorMeta]], None, None]:
    """Pack (name, tensor) pairs into uint8 buckets of at most ``bucket_bytes``; tensors larger than a bucket are
    split into chunks (``chunk_offset`` / ``chunk_size`` in the metadata)."""
    bucket = None
    metas: list[TensorMeta] = []
    used = 0
    for name, t in weights:
        raw = t.detach().contiguous().view(-1).view(torch.uint8)
        pos = 0
        while pos < raw.numel():
            if bucket is None:
                bucket = torch.empty(bucket_bytes, dtype=torch.uint8, device=device if device is not None else t.device)
                metas, used = [], 0
            take = min(raw.numel() - pos, bucket_bytes - used)
            bucket[used : used + take].copy_(raw[pos : pos + take])
            whole = take == raw.numel()
            metas.append(TensorMeta(name, tuple(t.shape), t.dtype, used, take, None if whole else pos, None if whole else raw.numel()))
            used += take
            pos += take
            if used == bucket_bytes:
                yield bucket, metas
                bucket = None
        # align the next tensor to 16 bytes
        if bucket is not None:
            used = min(bucket_bytes, (used + 15) // 16 * 16)
            if used == bucket_bytes:
                yield bucket, metas
                bucket = None
    if bucket is not None and metas:
        yield bucket, metas


class _ChunkAssembler:
    """Rebuilds tensors that were split over several buckets."""

    def __init__(self):
        self.partial: dict[str, tuple[torch.Tensor, int]] = {}

    def feed(self, bucket: torch.Tensor, metas: list[TensorMeta]):
        for m in metas:
            piece = bucket[m.offset : m.offset + m.nbytes]
            if m.chunk_offset is None:
                yield m.name, piece.clone().view(m.dtype).view(m.shape)
                continue
            buf, got = self.partial.get(m.name, (None, 0))
            if buf is None:
                buf = torch.empty(m.chunk_size, dtype=torch.uint8, device=bucket.device)
            buf[m.chunk_offset : m.chunk_offset + m.nbytes].copy_(piece)
            got += m.nbytes
            if got == m.chunk_size:
                self.partial.pop(m.name, None)
                yield m.name, buf.view(m.dtype).view(m.shape)
            else:
                self.partial[m.name] = (buf, got)


def split_weight_chunks(weights, bucket_bytes: int):
    return bucketize(weights, bucket_bytes)


def merge_weight_chunks(buckets):
    asm = _ChunkAssembler()
    for bucket, metas in buckets:
        yield from asm.feed(bucket, metas)


class CheckpointEngineManager:
    """Driver-side orchestration of a weight update across trainer workers and rollout replicas."""

    def __init__(self, config, trainer, replicas: Optional[list] = None):
        self.config = config
        self.backend = (config.get("backend", "naive") if hasattr(config, "get") else "naive")
        self.trainer = trainer  # worker group exposing update_weights()
        self.replicas = list(replicas or [])
        self.global_steps = 0

    def add_replicas(self, replicas: list) -> None:
        self.replicas.extend(replicas)

    def remove_replicas(self, replicas: list) -> None:
        self.replicas = [r for r in self.replicas if r not in replicas]

    async def _each(self, method: str, *args):
        await asyncio.gather(*[getattr(r, method)(*args) for r in self.replicas if hasattr(r, method)])

    def sleep_replicas(self) -> None:
        if self.replicas:
            asyncio.run(self._each("sleep"))

    def wake_up_replicas(self) -> None:
        if self.replicas:
            asyncio.run(self._each("wake_up"))

    def update_weights(self, global_steps: Optional[int] = None) -> dict:
        """abort in-flight generation -> trainer pushes weights (in place for ``naive``) -> clear KV -> resume."""
        t0 = time.time()
        if global_steps is not None:
            self.global_steps = global_steps
        if self.replicas:
            asyncio.run(self._each("abort_all_requests"))
        res = self.trainer.update_weights(self.global_steps)
        if self.replicas:
            asyncio.run(self._each("clear_kv_cache"))
            asyncio.run(self._each("resume_generation"))
        out = res[0] if isinstance(res, list) and res else (res or {})
        out = dict(out)
        out["timing_s/update_weights_total"] = time.time() - t0
        return out
