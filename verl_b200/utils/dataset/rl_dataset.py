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
                 data_source: str = "synthetic/mod7", image: Optional[dict] = None):
        """``image`` (vision-language runs without data files): ``{grid: [h, w] patches, merge_size, patch_dim,
        image_token_id, vision_start_token_id, vision_end_token_id}`` puts one random image in front of every prompt: its
        placeholder tokens into the ids and its patches ([h * w, patch_dim]) + grid into ``multi_modal_inputs``."""
        g = torch.Generator()
        g.manual_seed(seed)
        self.ids = torch.randint(vocab_low, vocab_high, (num_prompts, prompt_length), generator=g)
        self.data_source = data_source
        self.image = dict(image) if image else None
        self.seed = seed
        if self.image:
            h, w = (int(x) for x in self.image.get("grid", (4, 4)))
            m = int(self.image.get("merge_size", 2))
            n_tok = (h // m) * (w // m)
            assert n_tok + 2 < prompt_length, "the prompt is too short for the image placeholders"
            head = [int(self.image["vision_start_token_id"])] + [int(self.image["image_token_id"])] * n_tok + [int(self.image["vision_end_token_id"])]
            self.ids[:, : len(head)] = torch.tensor(head)

    def __len__(self) -> int:
        return self.ids.shape[0]

    def __getitem__(self, i: int) -> dict:
        ids = self.ids[i]
        out = {"input_ids": ids, "attention_mask": torch.ones_like(ids), "position_ids": torch.arange(ids.shape[0]),
               "data_source": self.data_source, "index": i,
               "reward_model": {"style": "rule", "ground_truth": int(ids[-1]) % 7 if self.image else int(ids[0]) % 7}}
        if self.image:
            h, w = (int(x) for x in self.image.get("grid", (4, 4)))
            g = torch.Generator()
            g.manual_seed(self.seed * 1000003 + i)
            out["multi_modal_inputs"] = {"pixel_values": torch.randn(h * w, int(self.image.get("patch_dim", 1176)), generator=g),
                                         "image_grid_thw": torch.tensor([[1, h, w]])}
        return out


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
        # vision-language rows: ``<image>`` / ``<video>`` marks in the prompt text refer to the entries of these columns
        self.image_key = g("image_key", "images")
        self.video_key = g("video_key", "videos")
        self.image_patch_size = int(g("image_patch_size", 14))
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
        if self.filter_overlong_prompts and self.tokenizer is not None and self.processor is None:
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

    def _has_media(self, row: dict) -> bool:
        def some(v):
            return v is not None and len(v) > 0

        return self.processor is not None and (some(row.get(self.image_key)) or some(row.get(self.video_key)))

    def _multimodal(self, row: dict, messages: list) -> tuple[torch.Tensor, torch.Tensor, dict, dict]:
        """Prompt ids with the processor's placeholder tokens, its tensors (``multi_modal_inputs``) and the prepared raw
        media (``multi_modal_data``, what an external inference server would be given)."""
        from .vision_utils import process_image, process_video

        structured = []
        for m in messages:
            content = m["content"]
            if isinstance(content, str):   # "<image>" / "<video>" marks split the text into typed segments
                parts = []
                for seg in re.split(r"(<image>|<video>)", content):
                    if seg == "<image>":
                        parts.append({"type": "image"})
                    elif seg == "<video>":
                        parts.append({"type": "video"})
                    elif seg:
                        parts.append({"type": "text", "text": seg})
                content = parts
            structured.append({"role": m["role"], "content": content})
        prompt = self.processor.apply_chat_template(structured, add_generation_prompt=True, tokenize=False,
                                                    **self.apply_chat_template_kwargs)
        data, kw = {}, {}
        imgs, vids = row.get(self.image_key), row.get(self.video_key)
        if imgs is not None and len(imgs) > 0:
            data["image"] = [process_image(im, self.image_patch_size) for im in imgs]
            kw["images"] = data["image"]
        if vids is not None and len(vids) > 0:
            data["video"] = [process_video(v, self.image_patch_size) for v in vids]
            kw["videos"] = data["video"]
        enc = dict(self.processor(text=[prompt], return_tensors="pt", **kw))
        ids, mask = enc.pop("input_ids"), enc.pop("attention_mask")
        enc.pop("second_per_grid_ts", None)
        return ids, mask, {k: v for k, v in enc.items() if isinstance(v, torch.Tensor)}, data

    def __getitem__(self, i: int) -> dict:
        row = dict(self.rows[i])
        messages = self._messages(row)
        mm_inputs = mm_data = None
        if self._has_media(row):
            ids, mask, mm_inputs, mm_data = self._multimodal(row, messages)
            assert ids.shape[1] <= self.max_prompt_length or self.truncation != "error", \
                f"prompt with media placeholders has {ids.shape[1]} tokens > max_prompt_length {self.max_prompt_length}"
        else:
            ids = torch.tensor(self._tokenize(messages), dtype=torch.int64).unsqueeze(0)
            mask = torch.ones_like(ids)
        pad = self.tokenizer.pad_token_id if getattr(self.tokenizer, "pad_token_id", None) is not None else 0
        ids, mask = VF.postprocess_data(ids, mask, self.max_prompt_length, pad, left_pad=True, truncation=self.truncation)
        out = {k: v for k, v in row.items() if k not in (self.prompt_key, self.image_key, self.video_key)}
        if self.processor is not None:   # every row of a vision-language dataset carries the fields (empty for text-only rows)
            out["multi_modal_inputs"], out["multi_modal_data"] = mm_inputs or {}, mm_data or {}
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
                                      seed=int(syn.get("seed", 0)) + (0 if is_train else 7919), image=syn.get("image"))
    return RLHFDataset(data_paths, tokenizer, data_config, processor, max_samples)


def create_rl_sampler(data_config, dataset, rank: int = 0, world: int = 1):
    if data_config.get("shuffle", True):
        return ShardedRandomSampler(len(dataset), seed=int(data_config.get("seed", 1) or 1), rank=rank, world=world)
    return ShardedSequentialSampler(len(dataset), rank=rank, world=world)
