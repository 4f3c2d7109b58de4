"""``BaseRollout`` adapter over the in-process :class:`RolloutEngine` (weights are shared with the trainer, so
``update_weights`` has nothing to copy unless the caller brings foreign tensors)."""

from __future__ import annotations

from typing import Generator

import torch

from ..base import BaseRollout
from .engine import RolloutEngine, SamplingParams

__all__ = ["NativeRollout"]


class NativeRollout(BaseRollout):
    def __init__(self, config, model_config, device_mesh=None, params=None):
        super().__init__(config, model_config, device_mesh)
        arch = model_config.arch if hasattr(model_config, "arch") else model_config
        assert params is not None, "NativeRollout shares the trainer's FlatParams"
        max_len = (config.max_model_len or (config.prompt_length + config.response_length)) + 1
        self.engine = RolloutEngine(arch, params, max_num_seqs=config.max_num_seqs, max_num_batched_tokens=config.max_num_batched_tokens,
                                    max_model_len=max_len, block_size=config.block_size,
                                    gpu_memory_utilization=config.gpu_memory_utilization, use_cuda_graph=not config.enforce_eager,
                                    sync_interval=config.sync_interval)

    async def resume(self, tags: list[str]):
        if "kv_cache" in tags:
            self.engine.resume_kv_cache()

    async def release(self):
        self.engine.release_kv_cache()

    async def update_weights(self, weights: Generator[tuple[str, torch.Tensor], None, None], **kwargs):
        views = dict(self.engine.params.hf_views())
        for name, t in weights:
            if name in views and views[name].data_ptr() != t.data_ptr():
                views[name].copy_(t.to(views[name].dtype))
        self.engine.clear_kv_cache()

    def generate(self, prompt_ids: list[list[int]], sampling_params: SamplingParams):
        return self.engine.generate(prompt_ids, sampling_params)
