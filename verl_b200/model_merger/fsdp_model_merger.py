"""Merges ``model_world_size_{W}_rank_{r}.pt`` shards into one HuggingFace state dict.

Two shard layouts are understood: this framework's flat layout (every rank holds a contiguous slice of one flat fp32
parameter buffer, plus the offset table that names the tensors inside it) and dictionaries of HF-named tensors sharded
along dim 0 (what FSDP ``SHARDED_STATE_DICT`` checkpoints of the reference contain once DTensors are made local).

Parity target: ``verl/model_merger/fsdp_model_merger.py`` (world-size discovery from file names / ``fsdp_config.json``,
parallel shard loading, dim-0 concatenation, bf16 cast).
"""

from __future__ import annotations

import json
import os
import re
from concurrent.futures import ThreadPoolExecutor

import torch

from .base_model_merger import BaseModelMerger

__all__ = ["FSDPModelMerger"]


class FSDPModelMerger(BaseModelMerger):
    def _world_size(self) -> int:
        cfg = os.path.join(self.config.local_dir, "fsdp_config.json")
        if os.path.exists(cfg):
            with open(cfg) as f:
                return int(json.load(f)["world_size"])
        for fn in os.listdir(self.config.local_dir):
            m = re.match(r"model_world_size_(\d+)_rank_0\.pt", fn)
            if m:
                return int(m.group(1))
        raise FileNotFoundError(f"no model_world_size_*_rank_0.pt under {self.config.local_dir}")

    def _load_shards(self, W: int) -> list[dict]:
        def one(r):
            return torch.load(os.path.join(self.config.local_dir, f"model_world_size_{W}_rank_{r}.pt"), map_location="cpu",
                              weights_only=False)

        with ThreadPoolExecutor(max_workers=min(32, W)) as ex:
            return list(ex.map(one, range(W)))

    def merge_state_dict(self) -> dict[str, torch.Tensor]:
        W = self._world_size()
        shards = self._load_shards(W)
        if "flat_shard" in shards[0]:
            return self._merge_flat(shards)
        out = {}
        for k in shards[0]:
            parts = [s[k] for s in shards]
            parts = [p.to_local() if hasattr(p, "to_local") else p for p in parts]
            same = all(p.shape == parts[0].shape for p in parts) and parts[0].dim() == 0
            out[k] = (parts[0] if same else torch.cat(parts, dim=0)).to(torch.bfloat16)
        return out

    def _merge_flat(self, shards: list[dict]) -> dict[str, torch.Tensor]:
        from ..models.config import ModelConfig
        from ..models.weights import FlatParams

        numel = int(shards[0]["numel"])
        flat = torch.zeros(numel, dtype=torch.float32)
        for s in shards:
            if s.get("layout") == "unit_sharded":  # zero_stage=3: a slice of every unit; (flat_lo, flat_hi, offset in the shard)
                for a, b, so in s["ranges"]:
                    flat[a:b] = s["flat_shard"][so : so + (b - a)].float()
                continue
            lo = int(s["shard_lo"])
            n = min(s["flat_shard"].numel(), numel - lo)
            flat[lo : lo + n] = s["flat_shard"][:n].float()
        arch = ModelConfig.from_pretrained(self.config.hf_model_config_path)
        value_head = False
        cfgp = os.path.join(self.config.local_dir, "fsdp_config.json")
        if os.path.exists(cfgp):
            with open(cfgp) as f:
                value_head = bool(json.load(f).get("value_head", False))
        from ..models import make_flat_params

        params = make_flat_params(arch, dtype=torch.float32, device="cpu", value_head=value_head or self.config.is_value_model,
                                  pad_to=len(shards), buffer=flat)
        out = {}
        for name, v in params.hf_views():
            if name == "lm_head.weight" and (arch.tie_word_embeddings or self.config.tie_word_embedding):
                continue
            out[name] = v.detach().to(torch.bfloat16).clone()
        return out
