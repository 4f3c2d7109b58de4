"""Preference pairs for reward-model training: every item is a (chosen, rejected) pair of prompt + response token
sequences, stacked as ``input_ids`` / ``attention_mask`` of shape [2, max_length] (index 0 = chosen).

Files are parquet (or json lines) with a prompt column and two response columns; remote paths are fetched into a local
cache by the first rank of a node while the others wait.
Parity target: ``verl/utils/dataset/rm_dataset.py`` (``RMDataset`` :40, ``download_files_distributed`` :26).
"""

from __future__ import annotations

import os
from typing import Optional, Union

import numpy as np
import torch
from torch.utils.data import Dataset

__all__ = ["RMDataset", "download_files_distributed"]


def download_files_distributed(download_fn) -> None:
    """Run ``download_fn`` on local rank 0 first (it fills the cache), then on everyone else (cache hits)."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        local_rank = int(os.environ.get("LOCAL_RANK", dist.get_rank()))
        if local_rank == 0:
            download_fn()
        dist.barrier()
        if local_rank != 0:
            download_fn()
    else:
        download_fn()


class RMDataset(Dataset):
    def __init__(self, parquet_files: Union[str, list[str]], tokenizer, prompt_key: str = "prompt", chosen_key: str = "chosen",
                 rejected_key: str = "rejected", max_length: int = 1024, add_eos: bool = True, cache_dir: str = "~/.cache/verl/rm",
                 max_samples: int = -1, shuffle: bool = False, seed: Optional[int] = None):
        self.files = [parquet_files] if isinstance(parquet_files, str) else list(parquet_files)
        if isinstance(tokenizer, str):
            from ..tokenizer import hf_tokenizer

            tokenizer = hf_tokenizer(tokenizer)
        self.tokenizer = tokenizer
        self.prompt_key, self.chosen_key, self.rejected_key = prompt_key, chosen_key, rejected_key
        self.max_length, self.add_eos = int(max_length), bool(add_eos)
        self.cache_dir = os.path.expanduser(cache_dir)
        self.max_samples, self.shuffle, self.seed = int(max_samples), shuffle, seed
        download_files_distributed(self._download)
        self._read()

    def _download(self) -> None:
        from ..fs import copy_to_local

        self.files = [copy_to_local(f, cache_dir=self.cache_dir) for f in self.files]

    def _read(self) -> None:
        import pandas as pd

        frames = [pd.read_json(f, lines=True) if f.endswith((".json", ".jsonl")) else pd.read_parquet(f) for f in self.files]
        df = pd.concat(frames, ignore_index=True)
        if 0 < self.max_samples < len(df):
            idx = (np.random.default_rng(self.seed).choice(len(df), self.max_samples, replace=False) if self.shuffle
                   else np.arange(self.max_samples))
            df = df.iloc[idx.tolist()]
        self.prompts = df[self.prompt_key].tolist()
        self.chosen = df[self.chosen_key].tolist()
        self.rejected = df[self.rejected_key].tolist()

    def __len__(self) -> int:
        return len(self.prompts)

    def _encode(self, text: str) -> list[int]:
        out = self.tokenizer(text, add_special_tokens=False) if callable(self.tokenizer) else self.tokenizer.encode(text)
        ids = out["input_ids"] if isinstance(out, dict) or hasattr(out, "keys") else out
        return [int(t) for t in ids]

    def _pad_to_length(self, ids: list[int]) -> tuple[torch.Tensor, torch.Tensor]:
        ids = ids[: self.max_length]
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        n = len(ids)
        input_ids = torch.tensor(ids + [pad] * (self.max_length - n), dtype=torch.long)
        mask = torch.cat([torch.ones(n, dtype=torch.long), torch.zeros(self.max_length - n, dtype=torch.long)])
        return input_ids, mask

    def __getitem__(self, item: int) -> dict:
        prompt = self._encode(self.prompts[item])
        eos = [self.tokenizer.eos_token_id] if self.add_eos and getattr(self.tokenizer, "eos_token_id", None) is not None else []
        pairs = [self._pad_to_length(prompt + self._encode(r) + eos) for r in (self.chosen[item], self.rejected[item])]
        return {"input_ids": torch.stack([p[0] for p in pairs]), "attention_mask": torch.stack([p[1] for p in pairs])}
