"""Skips expensive phases of a step by replaying what an earlier run dumped to disk (debugging the trainer without
paying for generation every time). ``@SkipManager.annotate("rollout")`` wraps a ``generate_sequences``-like method: when
a dump for the current step exists it is loaded and returned, otherwise the method runs and its result is dumped.

Before ``SkipManager.init(config)`` is called the decorators are inert.

Parity target: ``verl/utils/skip/skip_manager.py`` (190 lines: class-level state, ``init`` / ``set_step`` / ``annotate``)
and ``verl/utils/skip/base_skip.py`` (registry).
"""

from __future__ import annotations

import functools
from typing import Callable, Optional

__all__ = ["SkipManager", "SKIP_REGISTRY", "register_skip", "BaseSkip"]

SKIP_REGISTRY: dict[str, type] = {}


def register_skip(name: str):
    def deco(cls):
        SKIP_REGISTRY[name] = cls
        return cls

    return deco


class BaseSkip:
    def __init__(self, local_config, global_config):
        self.local_config, self.global_config = local_config, global_config

    def meet_precondition(self, step: int, func: Callable, *args, **kwargs) -> bool:
        return False

    def warp_function(self, step: int, func: Callable, *args, **kwargs):
        return func(*args, **kwargs)

    def prepare_data(self, step: int, result, *args, **kwargs) -> None:
        return None


class SkipManager:
    config = None
    step: int = -1
    skip_instances: dict = {}

    @classmethod
    def init(cls, config) -> None:
        from . import rollout_skip  # noqa: F401  (registers "rollout")

        skip_cfg = config.get("skip") if hasattr(config, "get") else getattr(config, "skip", None)
        cls.config, cls.step, cls.skip_instances = skip_cfg, -1, {}
        if not skip_cfg:
            return
        for name, skip_cls in SKIP_REGISTRY.items():
            local = skip_cfg.get(name) if hasattr(skip_cfg, "get") else getattr(skip_cfg, name, None)
            if local and (local.get("enable", False) if hasattr(local, "get") else getattr(local, "enable", False)):
                cls.skip_instances[name] = skip_cls(local, config)

    @classmethod
    def reset(cls) -> None:
        cls.config, cls.step, cls.skip_instances = None, -1, {}

    @classmethod
    def set_step(cls, step: int) -> None:
        cls.step = int(step)

    @classmethod
    def annotate(cls, name: str, step_fn: Optional[Callable[..., int]] = None):
        """Decorator factory. ``step_fn(*args, **kwargs)`` may extract the step from the call (async pipelines);
        otherwise the step set by ``set_step`` is used."""

        def deco(func):
            @functools.wraps(func)
            def wrapper(*args, **kwargs):
                inst = cls.skip_instances.get(name)
                if inst is None:
                    return func(*args, **kwargs)
                step = step_fn(*args, **kwargs) if step_fn is not None else cls.step
                if inst.meet_precondition(step, func, *args, **kwargs):
                    return inst.warp_function(step, func, *args, **kwargs)
                result = func(*args, **kwargs)
                inst.prepare_data(step, result, *args, **kwargs)
                return result

            return wrapper

        return deco
