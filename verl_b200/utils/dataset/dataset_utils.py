"""How SFT samples become a batch.

``DatasetPadMode`` says what a dataset hands out: ``no_padding`` (every sample at its own length), ``right`` or
``left_right`` (every sample already padded to a fixed length). ``SFTTensorCollator`` batches accordingly: fixed-length
samples are stacked; variable-length ones become jagged nested tensors (one row per sample, no padding stored), which the
packing engines consume directly; fields that are not tensors are kept as a list per key.

Parity target: ``verl/utils/dataset/dataset_utils.py`` (``DatasetPadMode`` :24, ``SFTTensorCollator`` :32-80).
"""

from __future__ import annotations

from enum import Enum
from typing import Any

import torch

__all__ = ["DatasetPadMode", "SFTTensorCollator", "pad_sample"]


class DatasetPadMode(str, Enum):
    RIGHT = "right"
    LEFT_RIGHT = "left_right"
    NO_PADDING = "no_padding"


def pad_sample(sample: dict, length: int, pad_token_id: int = 0) -> dict:
    """Right-pad the 1-D tensors of one sample to ``length`` (``input_ids`` with the pad id, masks and positions with 0) and
    add the ``attention_mask`` of the real tokens: what a dataset in ``right`` mode returns."""
    n = int(sample["input_ids"].shape[0])
    if n > length:
        raise ValueError(f"sample of {n} tokens does not fit the padded length {length}")
    out = {}
    for k, v in sample.items():
        if isinstance(v, torch.Tensor) and v.dim() == 1 and v.shape[0] == n:
            fill = pad_token_id if k == "input_ids" else 0
            out[k] = torch.cat([v, torch.full((length - n,), fill, dtype=v.dtype)])
        else:
            out[k] = v
    am = torch.zeros(length, dtype=torch.int64)
    am[:n] = 1
    out["attention_mask"] = am
    return out


class SFTTensorCollator:
    def __init__(self, pad_mode: DatasetPadMode = DatasetPadMode.LEFT_RIGHT):
        self.pad_mode = DatasetPadMode(pad_mode)

    def __call__(self, batch: list[dict[str, Any]]) -> dict[str, Any]:
        if self.pad_mode == DatasetPadMode.NO_PADDING:
            return self.collate_variable_batch(batch)
        return self.collate_fixed_batch(batch)

    @staticmethod
    def collate_fixed_batch(batch: list[dict[str, Any]]) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for key in batch[0]:
            vals = [item[key] for item in batch]
            if isinstance(vals[0], torch.Tensor):
                if any(v.shape != vals[0].shape for v in vals):
                    raise ValueError(f"field {key!r} has samples of different shapes: pad them in the dataset or use "
                                     f"pad_mode={DatasetPadMode.NO_PADDING.value}")
                out[key] = torch.stack(vals)
            elif isinstance(vals[0], (int, float, bool)):
                out[key] = torch.tensor(vals)
            else:
                out[key] = vals
        return out

    @staticmethod
    def collate_variable_batch(batch: list[dict[str, Any]]) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for key in sorted(set().union(*(d.keys() for d in batch))):
            vals = [item.get(key) for item in batch]
            if all(isinstance(v, torch.Tensor) for v in vals):
                # jagged layout: rows differ in their first dimension only (tokens; for 2-D fields like a 3-axis position
                # table stored [tokens, 3] the trailing sizes agree)
                out[key] = torch.nested.nested_tensor(vals, layout=torch.jagged) if vals[0].dim() >= 1 else torch.stack(vals)
            else:
                out[key] = vals
        return out
