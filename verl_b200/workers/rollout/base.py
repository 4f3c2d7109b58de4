"""Rollout interface and registry. Parity target: ``verl/workers/rollout/base.py`` (:29-109)."""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Generator, Optional

import torch

from ...protocol import DataProto

__all__ = ["BaseRollout", "get_rollout_class", "register_rollout", "_ROLLOUT_REGISTRY"]


class BaseRollout(ABC):
    """What a worker needs from an inference engine: generate, take new weights, hand memory back."""

    def __init__(self, config, model_config, device_mesh=None):
        self.config, self.model_config, self.device_mesh = config, model_config, device_mesh

    @abstractmethod
    async def resume(self, tags: list[str]):
        """Re-acquire device memory for ``weights`` and/or ``kv_cache``."""

    @abstractmethod
    async def release(self):
        """Give device memory back to the trainer."""

    @abstractmethod
    async def update_weights(self, weights: Generator[tuple[str, torch.Tensor], None, None], **kwargs):
        """Install new weights (name, tensor) pairs."""

    def generate_sequences(self, prompts: DataProto) -> DataProto:
        raise NotImplementedError


_ROLLOUT_REGISTRY: dict[tuple[str, str], str] = {
    ("native", "async"): "verl_b200.workers.rollout.native.adapter.NativeRollout",
    ("native", "sync"): "verl_b200.workers.rollout.native.adapter.NativeRollout",
    ("hf", "sync"): "verl_b200.workers.rollout.hf_rollout.HFRollout",
    ("naive", "sync"): "verl_b200.workers.rollout.naive_rollout.NaiveRollout",
}


def register_rollout(name: str, mode: str, fqn: str) -> None:
    _ROLLOUT_REGISTRY[(name, mode)] = fqn


def get_rollout_class(rollout_name: str, mode: str = "async") -> type[BaseRollout]:
    key = (rollout_name, mode)
    if key not in _ROLLOUT_REGISTRY:
        raise ValueError(f"Rollout {rollout_name} with mode {mode} is not supported (known: {sorted(_ROLLOUT_REGISTRY)})")
    import importlib

    mod, _, cls = _ROLLOUT_REGISTRY[key].rpartition(".")
    return getattr(importlib.import_module(mod), cls)
