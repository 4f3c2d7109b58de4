"""Conversions between padded [b, P+R] batches and jagged (no-padding) form.

Parity target: ``verl/workers/utils/padding.py`` (``left_right_2_no_padding`` :23-94, ``no_padding_2_padding``
:97-141 with the left-shift-by-one alignment, ``response_from_nested`` :194, ``response_to_nested`` :213).
"""

from __future__ import annotations

import torch

from ...utils.tensordict_lite import NestedRows, TensorDict

__all__ = ["left_right_2_no_padding", "no_padding_2_padding", "build_attention_mask_from_nested",
           "response_from_nested", "response_to_nested"]


def left_right_2_no_padding(data: TensorDict) -> TensorDict:
    """Strip padding: ``input_ids`` / ``position_ids`` / ``loss_mask`` become jagged rows; adds ``max_seq_len``,
    ``max_response_len`` and the per-row valid-token ``indices``."""
    ids, mask = data["input_ids"], data["attention_mask"].bool()
    R = data["responses"].shape[1]
    out = TensorDict({k: v for k, v in data.items()}, batch_size=data.batch_size)
    out["input_ids"] = NestedRows.from_padded(ids, mask)
    pos = data["position_ids"] if "position_ids" in data else (torch.cumsum(mask.long(), -1) - 1).clamp(min=0)
    out["position_ids"] = NestedRows.from_padded(pos, mask)
    resp_mask = data["response_mask"] if "response_mask" in data else data["attention_mask"][:, -R:]
    full_loss_mask = torch.cat([torch.zeros_like(ids[:, : ids.shape[1] - R]), resp_mask.to(ids.dtype)], dim=1)
    out["loss_mask"] = NestedRows.from_padded(full_loss_mask, mask)
    out["max_seq_len"] = int(ids.shape[1])
    out["max_response_len"] = int(R)
    out["indices"] = mask
    return out


def no_padding_2_padding(nested: NestedRows, data: TensorDict) -> torch.Tensor:
    """Per-token model outputs (jagged over full sequences) -> padded [b, R] response part.

    The output at position t predicts token t+1, so the response slice of sequence i is
    ``[seq_len - resp_len - 1, seq_len - 1)``."""
    R = int(data["max_response_len"]) if "max_response_len" in data else data["responses"].shape[1]
    resp_mask = data["response_mask"] if "response_mask" in data else data["attention_mask"][:, -R:]
    resp_len = resp_mask.sum(-1).long()
    b = len(nested)
    out = nested.values.new_zeros((b, R) + tuple(nested.values.shape[1:]))
    for i in range(b):
        row = nested.row(i)
        n, r = row.shape[0], int(resp_len[i])
        if r > 0:
            out[i, :r] = row[n - r - 1 : n - 1]
    return out


def build_attention_mask_from_nested(nested: NestedRows, max_len: int, left_pad_to: int | None = None) -> torch.Tensor:
    lens = nested.lengths()
    ar = torch.arange(max_len).unsqueeze(0)
    return (ar < lens.unsqueeze(1)).long()


def response_from_nested(nested: NestedRows, response_lens: torch.Tensor, max_response_len: int, pad_value=0) -> torch.Tensor:
    b = len(nested)
    out = nested.values.new_full((b, max_response_len), pad_value)
    for i in range(b):
        r = int(response_lens[i])
        if r:
            out[i, :r] = nested.row(i)[-r:]
    return out


def response_to_nested(padded: torch.Tensor, response_mask: torch.Tensor) -> NestedRows:
    return NestedRows.from_padded(padded, response_mask.bool())
