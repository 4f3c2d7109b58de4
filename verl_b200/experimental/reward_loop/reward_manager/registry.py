"""Name -> async reward manager class. Parity target: ``verl/experimental/reward_loop/reward_manager/registry.py``."""
from __future__ import annotations

__all__ = ["register", "get_reward_manager_cls", "REWARD_LOOP_MANAGERS"]

REWARD_LOOP_MANAGERS: dict[str, type] = {}


def register(name: str):
    def deco(cls):
        if name in REWARD_LOOP_MANAGERS and REWARD_LOOP_MANAGERS[name] is not cls:
            raise ValueError(f"reward manager '{name}' is already registered")
        REWARD_LOOP_MANAGERS[name] = cls
        return cls

    return deco


def get_reward_manager_cls(name: str) -> type:
    if name not in REWARD_LOOP_MANAGERS:
        raise ValueError(f"Unknown reward manager: {name} (known: {sorted(REWARD_LOOP_MANAGERS)})")
    return REWARD_LOOP_MANAGERS[name]
