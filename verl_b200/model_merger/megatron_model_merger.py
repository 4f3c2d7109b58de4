"""Merges a TP x PP sharded checkpoint of the tensor/pipeline-parallel engine into one HuggingFace state dict:
pipeline stages contribute disjoint layer ranges; within a stage, column-parallel tensors are concatenated along dim 0
(fused QKV and gate/up are first un-interleaved per rank), row-parallel tensors along dim 1, the rest is replicated.

Parity target: ``verl/model_merger/megatron_model_merger.py``.
"""

from __future__ import annotations

import os
import re

import torch

from .base_model_merger import BaseModelMerger

__all__ = ["MegatronModelMerger", "merge_tp_tensor"]

_ROW_PARALLEL = ("self_attn.o_proj.weight", "mlp.down_proj.weight")
_COL_PARALLEL = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "mlp.gate_proj", "mlp.up_proj", "embed_tokens.weight",
                 "lm_head.weight")


def merge_tp_tensor(name: str, parts: list[torch.Tensor]) -> torch.Tensor:
    if len(parts) == 1:
        return parts[0]
    if any(name.endswith(s) for s in _ROW_PARALLEL):
        return torch.cat(parts, dim=1)
    if any(s in name for s in _COL_PARALLEL):
        return torch.cat(parts, dim=0)
    return parts[0]


class MegatronModelMerger(BaseModelMerger):
    """Expects ``local_dir/mp_rank_{tp:02d}_{pp:03d}/model.pt`` files holding HF-named local tensors."""

    def merge_state_dict(self) -> dict[str, torch.Tensor]:
        ranks = {}
        for d in os.listdir(self.config.local_dir):
            m = re.match(r"mp_rank_(\d+)_(\d+)$", d)
            if m:
                ranks[(int(m.group(1)), int(m.group(2)))] = os.path.join(self.config.local_dir, d, "model.pt")
        if not ranks:
            raise FileNotFoundError(f"no mp_rank_XX_YYY directories under {self.config.local_dir}")
        tp = max(k[0] for k in ranks) + 1
        pp = max(k[1] for k in ranks) + 1
        out: dict[str, torch.Tensor] = {}
        for p in range(pp):
            shards = [torch.load(ranks[(t, p)], map_location="cpu", weights_only=False) for t in range(tp)]
            for name in shards[0]:
                out[name] = merge_tp_tensor(name, [s[name] for s in shards]).to(torch.bfloat16)
        return out
