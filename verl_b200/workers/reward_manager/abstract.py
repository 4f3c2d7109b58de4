"""Reward-manager interface. Parity target: ``verl/workers/reward_manager/abstract.py`` (72 lines)."""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Callable

import torch

from ...protocol import DataProto

__all__ = ["AbstractRewardManager", "RawRewardFn"]

RawRewardFn = Callable[..., Any]


class AbstractRewardManager(ABC):
    @abstractmethod
    def __init__(self, tokenizer: Any, num_examine: int, compute_score: RawRewardFn | None,
                 reward_fn_key: str = "data_source", **kwargs: Any):
        ...

    @abstractmethod
    def __call__(self, data: DataProto, return_dict: bool = False) -> torch.Tensor | dict[str, Any]:
        ...

    def _extract_reward_from_rm_scores(self, data: DataProto, return_dict: bool = False):
        if "rm_scores" not in data.batch.keys():
            return None
        if return_dict:
            keys = data.meta_info.get("reward_extra_keys", [])
            return {"reward_tensor": data.batch["rm_scores"],
                    "reward_extra_info": {k: data.non_tensor_batch[k] for k in keys}}
        return data.batch["rm_scores"]
