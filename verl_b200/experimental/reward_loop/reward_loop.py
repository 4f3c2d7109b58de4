"""Reward computation that runs alongside generation.

``RewardLoopWorker.compute_score`` decides per trajectory: a user reward function if configured (it may itself call the
reward-model router); else the discriminative reward model if one is enabled; else the rule-based default. The manager
fans a batch out over workers and assembles ``rm_scores`` (score on the last response token) plus the extra fields.

Parity target: ``verl/experimental/reward_loop/reward_loop.py`` (``migrate_legacy_reward_impl`` :39, ``RewardLoopWorker``
:93-270, ``RewardLoopManager`` :273-390).
"""

from __future__ import annotations

import asyncio
from typing import Any, Optional

import numpy as np
import torch

from ...protocol import DataProto
from .reward_manager import get_reward_manager_cls

__all__ = ["RewardLoopWorker", "RewardLoopManager", "migrate_legacy_reward_impl"]


def _get(node, key, default=None):
    if node is None:
        return default
    v = node.get(key, default) if hasattr(node, "get") else getattr(node, key, default)
    return default if v is None else v


def migrate_legacy_reward_impl(config):
    """Accept the older ``reward_model.*`` / top-level ``custom_reward_function`` layout: returns the unified view
    ``{"reward_manager", "custom_reward_function", "reward_model", "reward_kwargs", ...}``."""
    new = dict(_get(config, "reward", {}) or {})
    legacy = _get(config, "reward_model", {}) or {}
    new.setdefault("reward_manager", _get(legacy, "reward_manager", "naive"))
    new.setdefault("reward_kwargs", dict(_get(legacy, "reward_kwargs", {}) or {}))
    new.setdefault("custom_reward_function", dict(_get(config, "custom_reward_function", {}) or {}))
    rm = dict(_get(new, "reward_model", {}) or {})
    rm.setdefault("enable", bool(_get(legacy, "enable", False)))
    new["reward_model"] = rm
    return new


class RewardLoopWorker:
    def __init__(self, config, tokenizer=None, reward_router=None, reward_model_tokenizer=None, compute_score=None):
        self.config, self.tokenizer = config, tokenizer
        self.reward_router, self.reward_model_tokenizer = reward_router, reward_model_tokenizer
        self.rcfg = migrate_legacy_reward_impl(config)
        if compute_score is None and self.rcfg["custom_reward_function"].get("path"):
            from ...trainer.ppo.reward import get_custom_reward_fn

            compute_score = get_custom_reward_fn(config)
        self.custom = compute_score is not None
        cls = get_reward_manager_cls(str(self.rcfg.get("reward_manager", "naive")))
        self.reward_manager = cls(config, tokenizer, compute_score, reward_router_address=reward_router,
                                  reward_model_tokenizer=reward_model_tokenizer)

    async def compute_score(self, data: DataProto) -> dict:
        if not self.custom and self.rcfg["reward_model"].get("enable") and self.reward_router is not None:
            return await self.compute_score_disrm(data[-1:])
        return await self.reward_manager.run_single(data)

    async def compute_score_batch(self, data: DataProto) -> list[dict]:
        return list(await asyncio.gather(*[self.compute_score(data[i : i + 1]) for i in range(len(data))]))

    async def compute_score_disrm(self, data: DataProto) -> dict:
        item = data[0]
        am = item.batch["attention_mask"].bool()
        ids = item.batch["input_ids"][am].tolist()  # prompt + response without padding
        if self.reward_model_tokenizer is not None and self.tokenizer is not None and self.reward_model_tokenizer is not self.tokenizer:
            text = self.tokenizer.decode(ids, skip_special_tokens=False)  # re-tokenise for a reward model with another vocabulary
            ids = self.reward_model_tokenizer.encode(text)
        score = float(await self.reward_router.score(ids))
        return {"reward_score": score, "reward_extra_info": {"rm_score": score}}

    async def compute_score_for(self, out, kwargs: dict) -> Optional[float]:
        """Agent-loop hook: score one finished trajectory (``AgentLoopOutput``) before it is padded into a batch."""
        P, R = len(out.prompt_ids), len(out.response_ids)
        ids = torch.tensor([list(out.prompt_ids) + list(out.response_ids)], dtype=torch.int64)
        non = {}
        for k in ("data_source", "reward_model", "extra_info", "raw_prompt"):
            if k in kwargs:
                arr = np.empty(1, dtype=object)
                arr[0] = kwargs[k]
                non[k] = arr
        dp = DataProto.from_dict(tensors={"prompts": ids[:, :P], "responses": ids[:, P:], "input_ids": ids,
                                          "attention_mask": torch.ones_like(ids)}, non_tensors=non)
        res = await self.compute_score(dp)
        out.extra_fields.setdefault("reward_extra_info", {}).update(res.get("reward_extra_info", {}))
        return float(res["reward_score"])


class RewardLoopManager:
    def __init__(self, config, tokenizer=None, reward_router=None, num_workers: int = 1, **worker_kwargs):
        self.config = config
        self.workers = [RewardLoopWorker(config, tokenizer, reward_router, **worker_kwargs) for _ in range(max(1, num_workers))]

    @property
    def reward_loop_worker_handles(self) -> list[RewardLoopWorker]:
        return self.workers

    async def compute_rm_score_async(self, data: DataProto) -> DataProto:
        k = min(len(self.workers), max(1, len(data)))
        bounds = np.linspace(0, len(data), k + 1).astype(int)
        parts = await asyncio.gather(*[w.compute_score_batch(data[int(a):int(b)]) for w, a, b in zip(self.workers, bounds[:-1], bounds[1:]) if b > a])
        results = [r for part in parts for r in part]
        scores = [float(r["reward_score"]) for r in results]
        rm_scores = type(self.workers[0].reward_manager).assemble_rm_scores(data, scores)
        keys = sorted({k for r in results for k in r.get("reward_extra_info", {})})
        non = {}
        for key in keys:
            arr = np.empty(len(results), dtype=object)
            arr[:] = [r.get("reward_extra_info", {}).get(key) for r in results]
            non[key] = arr
        return DataProto.from_dict(tensors={"rm_scores": rm_scores}, non_tensors=non, meta_info={"reward_extra_keys": keys})

    def compute_rm_score(self, data: DataProto) -> DataProto:
        return asyncio.run(self.compute_rm_score_async(data))
