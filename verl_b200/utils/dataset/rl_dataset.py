"""Prompt datasets for RL: parquet/json chat data and synthetic random-token prompts.

Parity target: ``verl/utils/dataset/rl_dataset.py`` (``collate_fn`` :41, ``RLHFDataset`` :72-565: chat template,
prompt-length filter, left padding / truncation, extra fields for the reward function).
"""

from __future__ import annotations

import copy
import os
import re
from collections import defaultdict
from typing import Any, Optional

import numpy as np
import torch
from torch.utils.data import Dataset

from .. import torch_functional as VF
from .stateful import ShardedRandomSampler, ShardedSequentialSampler

__all__ = ["collate_fn", "RLHFDataset", "SyntheticPromptDataset", "create_rl_dataset", "create_rl_sampler"]


def collate_fn(data_list: list[dict]) -> dict:
    """Stack tensor fields; every other field becomes a numpy object array (one entry per row)."""
    tensors, non = defaultdict(list), defaultdict(list)
    for d in data_list:
        for k, v in d.items():
            (tensors if isinstance(v, torch.Tensor) else non)[k].append(v)
    out: dict[str, Any] = {k: torch.stack(v, dim=0) for k, v in tensors.items()}
    for k, v in non.items():
        arr = np.empty(len(v), dtype=object)
        arr[:] = v
        out[k] = arr
    return out


class SyntheticPromptDataset(Dataset):
    """``num_prompts`` prompts of ``prompt_length`` token ids drawn uniformly from [low, high)."""

    def __init__(self, num_prompts: int, prompt_length: int, vocab_low: int = 3, vocab_high: int = 512, seed: int = 0,
                 data_source: str = "synthetic/mod7"):
        g = torch.Generator()
        g.manual_seed(seed)
        self.ids = torch.randint(vocab_low, vocab_high, (num_prompts, prompt_length), generator=g)
        self.data_source = data_source

    def __len__(self) -> int:
        return self.ids.shape[0]

    def __getitem__(self, i: int) -> dict:
        ids = self.ids[i]
        return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "position_ids": torch.arange(ids.shape[0]),
                "data_source": self.data_source, "index": i,
                "reward_model": {"style": "rule", "ground_truth": int(ids[0]) % 7}}


class RLHFDataset(Dataset):
    """Chat prompts from parquet / json(l) files, tokenised with the chat template and left-padded."""

    def __init__(self, data_files, tokenizer, config, processor=None, max_samples: int = -1):
        if not isinstance(data_files, (list, tuple)):
            data_files = [data_files]
        self.data_files = [os.path.expanduser(str(f)) for f in data_files]
        self.tokenizer, self.processor, self.config = tokenizer, processor, config
        g = config.get
        self.prompt_key = g("prompt_key", "prompt")
        self.max_prompt_length = int(g("max_prompt_length", 1024))
        self.truncation = g("truncation", "error")
        self.filter_overlong_prompts = bool(g("filter_overlong_prompts", True))
        self.return_raw_chat = bool(g("return_raw_chat", False))
        self.return_full_prompt = bool(g("return_full_prompt", False))
        self.apply_chat_template_kwargs = dict(g("apply_chat_template_kwargs", {}) or {})
        self.need_tools_kwargs = bool(g("need_tools_kwargs", False))
        self.max_samples = max_samples
        self.seed = g("seed", None)
        self._read()

    def _read(self) -> None:
        import pandas as pd

        frames = []
        for f in self.data_files:
            if f.endswith(".parquet"):
                frames.append(pd.read_parquet(f))
            elif f.endswith(".jsonl") or f.endswith(".json"):
                frames.append(pd.read_json(f, lines=f.endswith(".jsonl")))
            else:
                raise ValueError(f"unsupported data file: {f}")
        df = pd.concat(frames, ignore_index=True)
        rows = df.to_dict("records")
        if self.max_samples and self.max_samples > 0:
            rng = np.random.RandomState(self.seed or 0)
            rows = [rows[i] for i in rng.permutation(len(rows))[: self.max_samples]]
        if self.filter_overlong_prompts and self.tokenizer is not None:
            rows = [r for r in rows if len(self._tokenize(self._messages(r))) <= self.max_prompt_length]
        self.rows = rows

    def _messages(self, row: dict):
        m = row[self.prompt_key]
        if isinstance(m, np.ndarray):
            m = m.tolist()
        if isinstance(m, str):
            m = [{"role": "user", "content": m}]
        return list(m)

    def _tokenize(self, messages) -> list[int]:
        tok = self.tokenizer
        if getattr(tok, "chat_template", None):
            text = tok.apply_chat_template(messages, add_generation_prompt=True, tokenize=False, **self.apply_chat_template_kwargs)
        else:
            text = "\n".join(f"{m['role']}: {m['content']}" for m in messages) + "\nassistant:"
        return tok(text, add_special_tokens=False)["input_ids"] if callable(tok) else tok.encode(text)

    def __len__(self) -> int:
        return len(self.rows)

    def __getitem__(self, i: int) -> dict:
        row = dict(self.rows[i])
        messages = self._messages(row)
        ids = torch.tensor(self._tokenize(messages), dtype=torch.int64).unsqueeze(0)
        mask = torch.ones_like(ids)
        pad = self.tokenizer.pad_token_id if getattr(self.tokenizer, "pad_token_id", None) is not None else 0
        ids, mask = VF.postprocess_data(ids, mask, self.max_prompt_length, pad, left_pad=True, truncation=self.truncation)
        out = {k: v for k, v in row.items() if k != self.prompt_key}
        out.update(input_ids=ids[0], attention_mask=mask[0], position_ids=VF.compute_position_id_with_mask(mask)[0])
        if self.return_raw_chat:
            out["raw_prompt"] = messages
        extra = out.get("extra_info") or {}
        out["index"] = extra.get("index", i) if isinstance(extra, dict) else i
        out.setdefault("data_source", "unknown")
        return out


def create_rl_dataset(data_paths, data_config, tokenizer, processor=None, is_train: bool = True, max_samples: int = -1):
    """Dataset factory: ``data.custom_cls`` (path + name) > ``data.synthetic`` > parquet/json files."""
    custom = data_config.get("custom_cls") or {}
    if custom.get("path"):
        from ..import_utils import load_extern_object

        cls = load_extern_object(custom["path"], custom["name"])
        return cls(data_files=data_paths, tokenizer=tokenizer, processor=processor, config=data_config)
    syn = data_config.get("synthetic")
    if syn or not data_paths:
        syn = syn or {}
        n = int(syn.get("num_prompts", data_config.get("train_batch_size", 8) * (4 if is_train else 1)))
        return SyntheticPromptDataset(n, int(syn.get("prompt_length", data_config.get("max_prompt_length", 32))),
                                      int(syn.get("vocab_low", 3)), int(syn.get("vocab_high", 512)),
                                      seed=int(syn.get("seed", 0)) + (0 if is_train else 7919))
    return RLHFDataset(data_paths, tokenizer, data_config, processor, max_samples)


def create_rl_sampler(data_config, dataset, rank: int = 0, world: int = 1):
    if data_config.get("shuffle", True):
        return ShardedRandomSampler(len(dataset), seed=int(data_config.get("seed", 1) or 1), rank=rank, world=world)
    return ShardedSequentialSampler(len(dataset), rank=rank, world=world)
