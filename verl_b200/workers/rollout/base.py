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
    ("naive", "sync"): "verl_b200.workers.rollout.naive.naive_rollout.NaiveRollout",
    # optional library back-end (import-gated); the native engine is the default and the measured path
    ("vllm", "async"): "verl_b200.workers.rollout.vllm_rollout.vllm_rollout.VLLMRollout",
    ("vllm", "sync"): "verl_b200.workers.rollout.vllm_rollout.vllm_rollout.VLLMRollout",
}

# engines of the reference's registry that this framework replaces with the native engine and does not wrap
_NOT_WRAPPED = {"sglang": "SGLang", "trtllm": "TensorRT-LLM"}


def register_rollout(name: str, mode: str, fqn: str) -> None:
    _ROLLOUT_REGISTRY[(name, mode)] = fqn


def get_rollout_class(rollout_name: str, mode: str = "async") -> type[BaseRollout]:
    key = (rollout_name, mode)
    if rollout_name in _NOT_WRAPPED and key not in _ROLLOUT_REGISTRY:
        raise ValueError(f"rollout.name={rollout_name}: {_NOT_WRAPPED[rollout_name]} is not embedded in the trainer's process by "
                         f"this framework; use rollout.name=native (built-in engine: continuous batching, paged KV, CUDA-graph "
                         f"decode), connect to a running server through the HTTP replicas (rollout.server_urls, "
                         f"workers/rollout/http_replica.py), or register an adapter with register_rollout()")
    if key not in _ROLLOUT_REGISTRY:
        raise ValueError(f"Rollout {rollout_name} with mode {mode} is not supported (known: {sorted(_ROLLOUT_REGISTRY)})")
    import importlib

    mod, _, cls = _ROLLOUT_REGISTRY[key].rpartition(".")
    return getattr(importlib.import_module(mod), cls)
