"""Model utilities: HF weight IO for the flat parameter store, position ids, parameter statistics.

Parity target: ``verl/utils/model.py`` (``compute_position_id_with_mask``, value-head model loading, HF
config surgery, weight loading helpers).
"""

from __future__ import annotations

import glob
import json
import os
from typing import Iterable

import torch

__all__ = ["load_hf_weights_into", "save_hf_weights", "compute_position_id_with_mask", "print_model_size",
           "get_model_size", "update_model_config", "load_valuehead_model"]


def compute_position_id_with_mask(mask: torch.Tensor) -> torch.Tensor:
    return torch.clip(torch.cumsum(mask, dim=-1) - 1, min=0, max=None)


def _iter_hf_tensors(path: str) -> Iterable[tuple[str, torch.Tensor]]:
    st_files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if st_files:
        from safetensors import safe_open

        for f in st_files:
            with safe_open(f, framework="pt", device="cpu") as sf:
                for k in sf.keys():
                    yield k, sf.get_tensor(k)
        return
    for f in sorted(glob.glob(os.path.join(path, "pytorch_model*.bin"))) + sorted(glob.glob(os.path.join(path, "*.pt"))):
        sd = torch.load(f, map_location="cpu", weights_only=True)
        yield from sd.items()


def load_hf_weights_into(params, path: str, strict: bool = False) -> list[str]:
    """Stream HF-named tensors from ``path`` (safetensors or torch files) into the fused flat storage."""
    views = dict(params.hf_views())
    seen = set()
    for name, t in _iter_hf_tensors(path):
        if name in views:
            views[name].copy_(t.to(views[name].dtype))
            seen.add(name)
    missing = [k for k in views if k not in seen and not (k == "lm_head.weight" and params.cfg.tie_word_embeddings)]
    if strict and missing:
        raise KeyError(f"missing tensors in {path}: {missing[:8]}")
    return missing


def save_hf_weights(params, path: str, max_shard_bytes: int = 5 << 30) -> None:
    """Write the working weights as HF safetensors shards + index (the "HF-merged" checkpoint layout)."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    shards, cur, cur_bytes = [], {}, 0
    for name, v in params.hf_views():
        if name == "lm_head.weight" and params.cfg.tie_word_embeddings:
            continue
        t = v.detach().to("cpu").contiguous().clone()
        nb = t.numel() * t.element_size()
        if cur and cur_bytes + nb > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[name] = t
        cur_bytes += nb
    if cur:
        shards.append(cur)
    index = {"metadata": {"total_size": 0}, "weight_map": {}}
    for i, sh in enumerate(shards):
        fn = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(path, fn), metadata={"format": "pt"})
        for k, t in sh.items():
            index["weight_map"][k] = fn
            index["metadata"]["total_size"] += t.numel() * t.element_size()
    if len(shards) > 1:
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump(index, f, indent=2)
    params.cfg.save_pretrained(path)


def get_model_size(params, scale: str = "auto"):
    n = sum(s.numel for s in params.specs)
    if scale == "auto":
        scale = "B" if n > 1e9 else "M" if n > 1e6 else "K" if n > 1e3 else ""
    div = {"B": 1e9, "M": 1e6, "K": 1e3, "": 1}[scale]
    return n / div, scale


def print_model_size(params, name: str = "model") -> None:
    n, s = get_model_size(params)
    print(f"{name} contains {n:.2f}{s} parameters")


def update_model_config(cfg, override: dict) -> None:
    for k, v in (override or {}).items():
        setattr(cfg, k, v)


def load_valuehead_model(model_config, device="cpu", dtype=torch.float32):
    """Flat parameter store with a scalar value head for critic / reward models."""
    from ..models import make_flat_params

    arch = model_config.arch if hasattr(model_config, "arch") else model_config
    return make_flat_params(arch, dtype=dtype, device=device, value_head=True)
