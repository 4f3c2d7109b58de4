"""Teacher models for on-policy distillation: frozen policies served next to the rollout replicas that answer
"what are your top-k next-token log-probs along this sequence?".

A ``TeacherServer`` wraps one frozen model; requests from many coroutines are batched (up to ``max_batch_tokens``
packed tokens per forward), the full-vocabulary logits are reduced to top-k chunk by chunk and only ``[len, k]``
ids / log-probs leave the device. ``TeacherModelManager`` owns the replicas of one teacher plus their load balancer;
``MultiTeacherModelManager`` maps teacher names (e.g. one per data source) to managers.

Parity target: ``verl/experimental/teacher_loop/teacher_model.py`` (``TeacherModelManager`` :37-163,
``MultiTeacherModelManager`` :165-215).
"""

from __future__ import annotations

import asyncio
from typing import Optional

import torch

from ...models.decoder import DecoderModel, PackedBatch
from ...workers.rollout.llm_server import GlobalRequestLoadBalancer

__all__ = ["TeacherServer", "TeacherModelManager", "MultiTeacherModelManager"]


class TeacherServer:
    def __init__(self, model: DecoderModel, topk: int = 64, max_batch_tokens: int = 16384, vocab_chunk_tokens: int = 2048):
        self.model, self.topk = model, int(topk)
        self.max_batch_tokens, self.chunk = int(max_batch_tokens), int(vocab_chunk_tokens)
        self._pending: list[tuple[list[int], asyncio.Future]] = []
        self._task: Optional[asyncio.Task] = None
        self.num_forwards = 0

    async def compute_topk_logprobs(self, token_ids: list[int], request_id: str = "") -> tuple[torch.Tensor, torch.Tensor]:
        """(ids [len-1, k] int64, logprobs [len-1, k] fp32) on CPU: row ``t`` is the teacher's prediction of token ``t+1``
        (its ``k`` most likely tokens; with ``topk=0`` one column: token ``t+1`` itself and its log-prob)."""
        fut = asyncio.get_running_loop().create_future()
        self._pending.append((list(token_ids), fut))
        if self._task is None:
            self._task = asyncio.ensure_future(self._drain())
        return await fut

    async def _drain(self) -> None:
        await asyncio.sleep(0)  # let concurrent callers enqueue so they share a forward
        while self._pending:
            batch, tokens = [], 0
            while self._pending and (not batch or tokens + len(self._pending[0][0]) <= self.max_batch_tokens):
                item = self._pending.pop(0)
                batch.append(item)
                tokens += len(item[0])
            try:
                outs = self._forward([ids for ids, _ in batch])
                for (_, fut), o in zip(batch, outs):
                    if not fut.done():
                        fut.set_result(o)
            except Exception as e:
                for _, fut in batch:
                    if not fut.done():
                        fut.set_exception(e)
            await asyncio.sleep(0)
        self._task = None

    @torch.no_grad()
    def _forward(self, seqs: list[list[int]]):
        dev = self.model.params.flat.device
        lens = [len(s) for s in seqs]
        flat = torch.tensor([t for s in seqs for t in s], dtype=torch.int64, device=dev)
        pb = PackedBatch.from_lengths(flat, lens, device=dev)
        self.num_forwards += 1
        hidden = self.model.forward_hidden(pb)
        W = self.model.params.lm_head_weight  # [V, H]
        ids_l, lps_l = [], []
        # topk == 0: the log-prob of the token that actually follows (what the sampled-token KL estimators need); the last row
        # of every sequence has no successor and is cut below, so the roll across sequence boundaries is harmless
        nxt = torch.roll(flat, -1)
        for lo in range(0, hidden.size(0), self.chunk):
            h = hidden[lo : lo + self.chunk]
            logits = (h @ W.t()).float()
            lp = torch.log_softmax(logits, -1)
            if self.topk <= 0:
                i = nxt[lo : lo + self.chunk, None]
                v = lp.gather(-1, i)
            else:
                v, i = torch.topk(lp, min(self.topk, lp.size(-1)), dim=-1)
            ids_l.append(i)
            lps_l.append(v)
        ids, lps = torch.cat(ids_l, 0).cpu(), torch.cat(lps_l, 0).cpu()
        outs, off = [], 0
        for n in lens:
            outs.append((ids[off : off + n - 1].clone(), lps[off : off + n - 1].clone()))
            off += n
        return outs


class TeacherModelManager:
    def __init__(self, name: str, servers: list[TeacherServer]):
        self.name = name
        self.servers = {f"inproc://teacher-{name}-{i}": s for i, s in enumerate(servers)}
        self.lb = GlobalRequestLoadBalancer(list(self.servers))

    @classmethod
    def from_models(cls, name: str, models: list[DecoderModel], topk: int = 64, **kw) -> "TeacherModelManager":
        return cls(name, [TeacherServer(m, topk=topk, **kw) for m in models])

    async def compute_topk_logprobs(self, request_id: str, token_ids: list[int]):
        sid = None
        while sid is None:
            sid = self.lb.acquire_server(request_id)
            if sid is None:
                await asyncio.sleep(0.01)
        try:
            return await self.servers[sid].compute_topk_logprobs(token_ids, request_id)
        finally:
            self.lb.release_server(sid)


class MultiTeacherModelManager:
    def __init__(self, managers: dict[str, TeacherModelManager], default: Optional[str] = None):
        assert managers, "at least one teacher"
        self.managers = dict(managers)
        self.default = default or next(iter(managers))

    def get_client(self) -> dict[str, TeacherModelManager]:
        return self.managers

    def resolve(self, routing_key: Optional[str]) -> TeacherModelManager:
        return self.managers.get(str(routing_key), self.managers[self.default])
