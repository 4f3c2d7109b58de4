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
    """Folds the shards of a model-parallel checkpoint into HF tensors. Layout schema v2 keeps them under
    ``local_dir/model/dist_ckpt/mp_rank_{tp:02d}_{pp:03d}[_{ep:03d}]/model.pt`` (``ckpt_contents.json`` names the place);
    a directory of the earlier flat layout (``mp_rank_*`` at the root) is read as well."""

    def _shard_root(self) -> str:
        root = self.config.local_dir
        man = os.path.join(root, "ckpt_contents.json")
        if os.path.exists(man):
            import json

            with open(man) as f:
                contents = json.load(f).get("contents", {})
            if "model" not in contents:
                raise FileNotFoundError(f"{man} lists no model shards (saved: {sorted(contents)})")
            return os.path.join(root, contents["model"]["path"])
        return root

    def merge_state_dict(self) -> dict[str, torch.Tensor]:
        root = self._shard_root()
        ranks = {}
        for d in os.listdir(root):
            m = re.match(r"mp_rank_(\d+)_(\d+)(?:_(\d+))?$", d)
            if m:
                ranks[(int(m.group(1)), int(m.group(2)), int(m.group(3) or 0))] = os.path.join(root, d, "model.pt")
        if not ranks:
            raise FileNotFoundError(f"no mp_rank_XX_YYY directories under {root}")
        tp = max(k[0] for k in ranks) + 1
        pp = max(k[1] for k in ranks) + 1
        ep = max(k[2] for k in ranks) + 1
        first = torch.load(next(iter(ranks.values())), map_location="cpu", weights_only=False)
        if "__shard_meta__" in first:
            return self._merge_with_shard_meta(ranks, tp, pp, ep)
        # shards stored under HF names (no placement record): the naming rules decide
        out: dict[str, torch.Tensor] = {}
        for p in range(pp):
            shards = [torch.load(ranks[(t, p, 0)], map_location="cpu", weights_only=False) for t in range(tp)]
            for name in shards[0]:
                out[name] = merge_tp_tensor(name, [s[name] for s in shards]).to(torch.bfloat16)
        return out

    def _merge_with_shard_meta(self, ranks: dict, tp: int, pp: int, ep: int) -> dict[str, torch.Tensor]:
        """Every shard file records how its tensors sit in the unsharded ones (replicated, row blocks, columns, experts): the
        shards are written into a full-layout parameter buffer and read back under their HF names."""
        import json

        from ..models import make_flat_params
        from ..models.config import ModelConfig
        from ..parallel.model_parallel import ShardMap, _slices, cat_dim

        arch = ModelConfig.from_pretrained(self.config.hf_model_config_path)
        value_head = self.config.is_value_model
        man = os.path.join(self.config.local_dir, "ckpt_contents.json")
        if os.path.exists(man):
            with open(man) as f:
                value_head = value_head or bool(json.load(f).get("backend", {}).get("value_head", False))
        full = make_flat_params(arch, dtype=torch.float32, device="cpu", value_head=value_head)
        seen = set()
        for (t, p, e), path in sorted(ranks.items()):
            shard = torch.load(path, map_location="cpu", weights_only=False)
            meta = shard.pop("__shard_meta__")
            for name, local in shard.items():
                if name not in full.views:
                    continue
                kind, blocks = meta[name]
                parts = _slices(ShardMap(name, name, kind, tuple(blocks)), full.views[name], tp, t, ep, e)
                off, dim = 0, cat_dim(kind)
                for part in parts:
                    n = part.shape[dim] if len(parts) > 1 else local.shape[dim] if local.dim() > dim else 0
                    part.copy_((local.narrow(dim, off, n) if len(parts) > 1 else local).float())
                    off += n
                seen.add(name)
        missing = [n for n in full.views if n not in seen]
        if missing:
            raise RuntimeError(f"checkpoint shards do not cover {missing[:5]}{' ...' if len(missing) > 5 else ''}")
        out = {}
        for name, v in full.hf_views():
            if name == "lm_head.weight" and (arch.tie_word_embeddings or self.config.tie_word_embedding):
                continue
            out[name] = v.to(torch.bfloat16).clone()
        return out
