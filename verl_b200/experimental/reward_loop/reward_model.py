"""Discriminative reward models served next to the rollout replicas: a decoder with a scalar value head scores a whole
conversation by the value at its last token. Concurrent requests are packed into one forward.

Parity target: ``verl/experimental/reward_loop/reward_model.py`` (``RewardModelManager``: standalone replicas + router).
"""

from __future__ import annotations

import asyncio
from typing import Optional

import torch

from ...models.decoder import DecoderModel, PackedBatch
from .router import NaiveRouter

__all__ = ["RewardModelServer", "RewardModelManager"]


class RewardModelServer:
    def __init__(self, model: DecoderModel, max_batch_tokens: int = 32768):
        assert model.params.value_head, "a discriminative reward model needs a value head"
        self.model, self.max_batch_tokens = model, int(max_batch_tokens)
        self._pending: list = []
        self._task: Optional[asyncio.Task] = None
        self.num_forwards = 0

    async def score(self, token_ids: list[int], **kw) -> float:
        fut = asyncio.get_running_loop().create_future()
        self._pending.append((list(token_ids), fut))
        if self._task is None:
            self._task = asyncio.ensure_future(self._drain())
        return await fut

    async def _drain(self) -> None:
        await asyncio.sleep(0)
        while self._pending:
            batch, tokens = [], 0
            while self._pending and (not batch or tokens + len(self._pending[0][0]) <= self.max_batch_tokens):
                batch.append(self._pending.pop(0))
                tokens += len(batch[-1][0])
            try:
                vals = self._forward([ids for ids, _ in batch])
                for (_, fut), v in zip(batch, vals):
                    if not fut.done():
                        fut.set_result(v)
            except Exception as e:
                for _, fut in batch:
                    if not fut.done():
                        fut.set_exception(e)
            await asyncio.sleep(0)
        self._task = None

    @torch.no_grad()
    def _forward(self, seqs: list[list[int]]) -> list[float]:
        dev = self.model.params.flat.device
        lens = [len(s) for s in seqs]
        flat = torch.tensor([t for s in seqs for t in s], dtype=torch.int64, device=dev)
        pb = PackedBatch.from_lengths(flat, lens, device=dev)
        self.num_forwards += 1
        values = self.model.forward_values(pb, need_grad=False).float()
        last = (pb.cu_seqlens[1:].long() - 1).to(values.device)
        return values[last].cpu().tolist()


class RewardModelManager:
    def __init__(self, servers: list[RewardModelServer]):
        self.servers = servers
        self.router = NaiveRouter(servers)

    @classmethod
    def from_models(cls, models: list[DecoderModel], **kw) -> "RewardModelManager":
        return cls([RewardModelServer(m, **kw) for m in models])

    def get_router_address(self):
        return self.router
