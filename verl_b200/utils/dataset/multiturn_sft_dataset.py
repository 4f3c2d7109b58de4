"""Multi-turn SFT data: chat messages -> token ids with a loss mask over assistant tokens only.

Parity target: ``verl/utils/dataset/multiturn_sft_dataset.py`` (456 lines): per-message incremental tokenisation
so that the loss mask follows assistant turns exactly, truncation, optional tools, no-padding output.
"""

from __future__ import annotations

from typing import Any, Optional

import numpy as np
import torch
from torch.utils.data import Dataset

__all__ = ["MultiTurnSFTDataset", "SyntheticSFTDataset", "sft_collate"]


class SyntheticSFTDataset(Dataset):
    """Random token sequences with a random prompt/response split (for benchmarks and tests)."""

    def __init__(self, num_samples: int, max_length: int, vocab_size: int, seed: int = 0, min_length: int = 8):
        g = torch.Generator()
        g.manual_seed(seed)
        self.lens = torch.randint(min_length, max_length + 1, (num_samples,), generator=g)
        self.ids = [torch.randint(3, vocab_size, (int(n),), generator=g) for n in self.lens]
        self.split = [int(torch.randint(1, int(n), (1,), generator=g)) for n in self.lens]

    def __len__(self):
        return len(self.ids)

    def __getitem__(self, i):
        ids = self.ids[i]
        mask = torch.zeros_like(ids)
        mask[self.split[i]:] = 1
        return {"input_ids": ids, "loss_mask": mask, "position_ids": torch.arange(ids.shape[0])}


class MultiTurnSFTDataset(Dataset):
    def __init__(self, parquet_files, tokenizer, config=None, max_samples: int = -1):
        import pandas as pd

        config = config or {}
        files = parquet_files if isinstance(parquet_files, (list, tuple)) else [parquet_files]
        frames = [pd.read_parquet(f) if str(f).endswith(".parquet") else pd.read_json(f, lines=str(f).endswith(".jsonl"))
                  for f in files]
        df = pd.concat(frames, ignore_index=True)
        self.tokenizer = tokenizer
        self.messages_key = config.get("messages_key", "messages")
        self.tools_key = config.get("tools_key", "tools")
        self.max_length = int(config.get("max_length", 1024))
        self.truncation = config.get("truncation", "error")
        self.rows = df.to_dict("records")
        if max_samples and max_samples > 0:
            self.rows = self.rows[:max_samples]

    def __len__(self):
        return len(self.rows)

    def _render(self, messages, tools=None, add_generation_prompt: bool = False) -> list[int]:
        tok = self.tokenizer
        kw = {"tools": tools} if tools else {}
        if getattr(tok, "chat_template", None):
            return tok.apply_chat_template(messages, tokenize=True, add_generation_prompt=add_generation_prompt, **kw)
        text = "".join(f"<|{m['role']}|>{m['content']}\n" for m in messages) + ("<|assistant|>" if add_generation_prompt else "")
        return tok.encode(text, add_special_tokens=False)

    def __getitem__(self, i) -> dict[str, Any]:
        row = self.rows[i]
        messages = row[self.messages_key]
        messages = messages.tolist() if isinstance(messages, np.ndarray) else list(messages)
        tools = row.get(self.tools_key)
        ids: list[int] = []
        mask: list[int] = []
        for t, msg in enumerate(messages):
            # tokens contributed by turn t = render(messages[:t+1]) minus render(messages[:t]); for assistant turns the
            # generation prompt belongs to the (unmasked-out) context, the content and end-of-turn to the loss
            upto = self._render(messages[: t + 1], tools)
            if msg["role"] == "assistant":
                ctx = self._render(messages[:t], tools, add_generation_prompt=True)
                new_ctx = ctx[len(ids):]
                ids += new_ctx
                mask += [0] * len(new_ctx)
                new = upto[len(ids):]
                ids += new
                mask += [1] * len(new)
            else:
                new = upto[len(ids):]
                ids += new
                mask += [0] * len(new)
        if len(ids) > self.max_length:
            if self.truncation == "error":
                raise ValueError(f"sequence of {len(ids)} tokens exceeds max_length={self.max_length}")
            sl = slice(0, self.max_length) if self.truncation == "right" else slice(len(ids) - self.max_length, None)
            ids, mask = ids[sl], mask[sl]
        ids_t = torch.tensor(ids, dtype=torch.int64)
        return {"input_ids": ids_t, "loss_mask": torch.tensor(mask, dtype=torch.int64), "position_ids": torch.arange(len(ids))}


def sft_collate(items: list[dict], pad_token_id: int = 0) -> dict:
    """Right-pad to the longest sample; the batch is expressed in the trainer's (prompt=1 token, response=rest)
    convention so the packed engine path (labels = next token, loss on masked positions) applies unchanged."""
    L = max(int(x["input_ids"].shape[0]) for x in items)
    b = len(items)
    ids = torch.full((b, L), pad_token_id, dtype=torch.int64)
    am = torch.zeros(b, L, dtype=torch.int64)
    lm = torch.zeros(b, L, dtype=torch.int64)
    for i, x in enumerate(items):
        n = x["input_ids"].shape[0]
        ids[i, :n] = x["input_ids"]
        am[i, :n] = 1
        lm[i, :n] = x["loss_mask"]
    # response part = tokens 1..L-1 (their log-probs come from positions 0..L-2)
    out = {"input_ids": ids, "attention_mask": am, "position_ids": (am.cumsum(-1) - 1).clamp(min=0),
           "responses": ids[:, 1:], "response_mask": lm[:, 1:] * am[:, 1:]}
    if any("multi_modal_inputs" in x for x in items):   # vision-language samples: the processor's tensors stay per row
        out["multi_modal_inputs"] = [x.get("multi_modal_inputs") or {} for x in items]
    return out
