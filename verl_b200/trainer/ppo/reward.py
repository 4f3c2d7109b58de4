"""Reward plumbing: custom reward functions, reward-manager loading, score extraction.

Parity target: ``verl/trainer/ppo/reward.py`` (``get_custom_reward_fn`` :50, ``load_reward_manager`` :111,
``extract_reward`` :160).
"""

from __future__ import annotations

import inspect
from functools import partial
from typing import Any, Optional

import torch

from ...protocol import DataProto
from ...utils.import_utils import load_extern_object
from ...utils.reward_score import default_compute_score
from ...workers.reward_manager import get_reward_manager_cls

__all__ = ["get_custom_reward_fn", "load_reward_manager", "compute_reward", "extract_reward"]


def get_custom_reward_fn(config) -> Optional[Any]:
    """The user function named by ``custom_reward_function.{path,name}`` (None when unset)."""
    node = config.get("custom_reward_function") or (config.get("reward") or {}).get("custom_reward_function") or {}
    path = node.get("path")
    if not path:
        return None
    fn = load_extern_object(path, node.get("name", "compute_score"))
    kw = dict(node.get("reward_kwargs", {}) or {})
    if not kw:
        return fn
    if inspect.iscoroutinefunction(fn):
        async def wrapped(*a, **k):
            return await fn(*a, **k, **kw)

        return wrapped
    return partial(fn, **kw)


def load_reward_manager(config, tokenizer, num_examine: int = 0, **reward_kwargs):
    rm_cfg = config.get("reward_model") or (config.get("reward") or {}).get("reward_manager") or {}
    name = rm_cfg.get("reward_manager", rm_cfg.get("name", "naive")) if hasattr(rm_cfg, "get") else "naive"
    custom = get_custom_reward_fn(config)
    cls = get_reward_manager_cls(name)
    extra = dict(rm_cfg.get("reward_kwargs", {}) or {}) if hasattr(rm_cfg, "get") else {}
    extra.update(reward_kwargs)
    return cls(tokenizer=tokenizer, num_examine=num_examine, compute_score=custom or default_compute_score,
               reward_fn_key=config.data.get("reward_fn_key", "data_source"), **extra)


def compute_reward(data: DataProto, reward_fn) -> tuple[torch.Tensor, dict]:
    try:
        res = reward_fn(data, return_dict=True)
        return res["reward_tensor"], res.get("reward_extra_info", {})
    except TypeError:
        return reward_fn(data), {}


def extract_reward(data: DataProto) -> tuple[torch.Tensor, dict]:
    keys = data.meta_info.get("reward_extra_keys", [])
    return data.batch["rm_scores"], {k: data.non_tensor_batch[k] for k in keys}
