"""Reward-manager registry. Parity target: ``verl/workers/reward_manager/registry.py`` (55 lines)."""

from __future__ import annotations

from typing import Callable

__all__ = ["register", "get_reward_manager_cls", "REWARD_MANAGER_REGISTRY"]

REWARD_MANAGER_REGISTRY: dict[str, type] = {}


def register(name: str) -> Callable[[type], type]:
    def deco(cls: type) -> type:
        if name in REWARD_MANAGER_REGISTRY and REWARD_MANAGER_REGISTRY[name] is not cls:
            raise ValueError(f"Reward manager {name} has already been registered: {REWARD_MANAGER_REGISTRY[name]} vs {cls}")
        REWARD_MANAGER_REGISTRY[name] = cls
        return cls

    return deco


def get_reward_manager_cls(name: str) -> type:
    if name not in REWARD_MANAGER_REGISTRY:
        raise ValueError(f"Unknown reward manager: {name}")
    return REWARD_MANAGER_REGISTRY[name]
