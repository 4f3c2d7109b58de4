"""Async reward managers score ONE trajectory per call (``run_single``) so that scoring overlaps generation.

Parity target: ``verl/experimental/reward_loop/reward_manager/base.py:35-82``.
"""

from __future__ import annotations

import asyncio
import inspect
from abc import ABC, abstractmethod
from typing import Any, Callable, Optional

import torch

from ....protocol import DataProto

__all__ = ["RewardManagerBase"]


class RewardManagerBase(ABC):
    def __init__(self, config, tokenizer, compute_score: Optional[Callable[..., Any]] = None, reward_router_address=None,
                 reward_model_tokenizer=None):
        from ....utils.reward_score import default_compute_score

        self.config, self.tokenizer = config, tokenizer
        self.compute_score = compute_score or default_compute_score
        self.is_async_reward_score = inspect.iscoroutinefunction(self.compute_score)
        self.reward_router_address, self.reward_model_tokenizer = reward_router_address, reward_model_tokenizer

    @abstractmethod
    async def run_single(self, data: DataProto) -> dict:
        """``{"reward_score": float, "reward_extra_info": dict}`` for a one-row batch."""

    # ---- helpers shared by the managers
    def _unpack(self, data: DataProto):
        item = data[-1:][0]  # multi-sequence outputs are judged by their last sequence
        resp = item.batch["responses"]
        R = resp.shape[-1]
        n = int(item.batch["attention_mask"][-R:].sum())
        ids = resp[:n]
        nt = item.non_tensor_batch
        rm = nt.get("reward_model") or {}
        extra = dict(nt.get("extra_info") or {})
        return ids, n, nt.get("data_source", "unknown"), (rm.get("ground_truth") if isinstance(rm, dict) else rm), extra, item

    def _decode(self, ids) -> str:
        if self.tokenizer is None:
            return " ".join(str(int(t)) for t in ids)
        return self.tokenizer.decode(ids, skip_special_tokens=True)

    async def _score(self, **kw):
        if self.reward_router_address is not None:
            kw.update(reward_router_address=self.reward_router_address, reward_model_tokenizer=self.reward_model_tokenizer)
        if self.is_async_reward_score:
            return await self.compute_score(**kw)
        return await asyncio.get_running_loop().run_in_executor(None, lambda: self.compute_score(**kw))

    @classmethod
    def assemble_rm_scores(cls, data: DataProto, scores: list[float]) -> torch.Tensor:
        """[b, R] tensor with each score on the last valid response token."""
        P = data.batch["prompts"].size(1)
        n = data.batch["attention_mask"][:, P:].sum(1)
        out = torch.zeros_like(data.batch["responses"], dtype=torch.float32)
        out[torch.arange(out.size(0)), (n - 1).clamp_min(0)] = out.new_tensor(scores)
        return out
