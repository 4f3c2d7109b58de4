"""Checkpoint merging: turn the sharded training checkpoint of a run into a HuggingFace-format model directory
(``merge``), or check a merged model against a reference one tensor by tensor (``test``).

Parity target: ``verl/model_merger/base_model_merger.py`` (``ModelMergerConfig``, ``BaseModelMerger.save_hf_model_and_tokenizer``,
``parse_args``) and ``verl/model_merger/__main__.py``.
"""

from __future__ import annotations

import argparse
import os
import shutil
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Optional

import torch

__all__ = ["ModelMergerConfig", "BaseModelMerger", "parse_args"]


@dataclass
class ModelMergerConfig:
    operation: str                     # merge | test
    backend: str                       # fsdp | megatron
    local_dir: str                     # .../global_step_N/actor
    target_dir: Optional[str] = "tmp"
    hf_model_config_path: Optional[str] = None
    test_hf_dir: Optional[str] = None
    tie_word_embedding: bool = False
    trust_remote_code: bool = False
    is_value_model: bool = False
    use_cpu_initialization: bool = False
    private: bool = False
    hf_upload_path: Optional[str] = None

    def __post_init__(self):
        if self.hf_model_config_path is None:
            self.hf_model_config_path = os.path.join(self.local_dir, "huggingface")
        if self.operation == "test":
            self.target_dir = None


class BaseModelMerger(ABC):
    def __init__(self, config: ModelMergerConfig):
        self.config = config

    @abstractmethod
    def merge_state_dict(self) -> dict[str, torch.Tensor]:
        """HF-named tensors of the full model."""

    def save_hf_model_and_tokenizer(self, state_dict: dict[str, torch.Tensor]) -> None:
        from safetensors.torch import save_file

        out = self.config.target_dir
        os.makedirs(out, exist_ok=True)
        shards, cur, size = [], {}, 0
        for k, v in state_dict.items():
            nb = v.numel() * v.element_size()
            if cur and size + nb > (5 << 30):
                shards.append(cur)
                cur, size = {}, 0
            cur[k] = v.contiguous()
            size += nb
        if cur:
            shards.append(cur)
        index = {"metadata": {"total_size": sum(v.numel() * v.element_size() for v in state_dict.values())}, "weight_map": {}}
        for i, sh in enumerate(shards):
            fn = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            save_file(sh, os.path.join(out, fn), metadata={"format": "pt"})
            index["weight_map"].update({k: fn for k in sh})
        if len(shards) > 1:
            import json

            with open(os.path.join(out, "model.safetensors.index.json"), "w") as f:
                json.dump(index, f, indent=1)
        src = self.config.hf_model_config_path
        if src and os.path.isdir(src):  # config.json, tokenizer files, generation config travel along
            for fn in os.listdir(src):
                if not fn.endswith((".safetensors", ".bin", ".pt")) and os.path.isfile(os.path.join(src, fn)):
                    shutil.copy2(os.path.join(src, fn), os.path.join(out, fn))

    def _test_state_dict(self, state_dict: dict[str, torch.Tensor]) -> None:
        from ..utils.model import _iter_hf_tensors

        ref = dict(_iter_hf_tensors(self.config.test_hf_dir))
        missing = set(ref) - set(state_dict)
        extra = set(state_dict) - set(ref)
        assert not missing and not extra, f"key mismatch: missing {sorted(missing)[:5]} extra {sorted(extra)[:5]}"
        for k, v in ref.items():
            assert v.shape == state_dict[k].shape, f"{k}: shape {tuple(state_dict[k].shape)} vs {tuple(v.shape)}"
            torch.testing.assert_close(state_dict[k].to(v.dtype), v, atol=1e-6, rtol=1e-6)

    def merge_and_save(self) -> None:
        sd = self.merge_state_dict()
        if self.config.operation == "test":
            self._test_state_dict(sd)
        elif self.config.operation == "merge":
            self.save_hf_model_and_tokenizer(sd)
            if self.config.hf_model_config_path and os.path.isdir(self.config.hf_model_config_path):
                from .output_validation import validate_hf_model_output

                validate_hf_model_output(self.config.target_dir)   # a half-written output fails here, not at its first load
        else:
            raise ValueError(f"Unknown operation: {self.config.operation}")

    def cleanup(self) -> None:
        return None


def parse_args(argv=None) -> ModelMergerConfig:
    p = argparse.ArgumentParser(description="verl_b200 model merger")
    sub = p.add_subparsers(dest="operation", required=True)
    base = argparse.ArgumentParser(add_help=False)
    base.add_argument("--backend", choices=["fsdp", "megatron"], required=True)
    base.add_argument("--local_dir", required=True)
    base.add_argument("--tie-word-embedding", action="store_true")
    base.add_argument("--trust-remote-code", action="store_true")
    base.add_argument("--is-value-model", action="store_true")
    base.add_argument("--use_cpu_initialization", action="store_true")
    m = sub.add_parser("merge", parents=[base])
    m.add_argument("--target_dir", default="tmp")
    m.add_argument("--hf_upload_path", default=None)
    m.add_argument("--private", action="store_true")
    t = sub.add_parser("test", parents=[base])
    t.add_argument("--test_hf_dir", required=True)
    a = p.parse_args(argv)
    return ModelMergerConfig(operation=a.operation, backend=a.backend, local_dir=a.local_dir,
                             target_dir=getattr(a, "target_dir", None), test_hf_dir=getattr(a, "test_hf_dir", None),
                             tie_word_embedding=a.tie_word_embedding, trust_remote_code=a.trust_remote_code,
                             is_value_model=a.is_value_model, use_cpu_initialization=a.use_cpu_initialization,
                             private=getattr(a, "private", False), hf_upload_path=getattr(a, "hf_upload_path", None))
