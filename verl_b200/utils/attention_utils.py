"""Padding <-> packed conversions around variable-length attention.

Parity target: ``verl/utils/attention_utils.py:23-150`` (``index_first_axis``, ``pad_input``, ``unpad_input``,
``rearrange``; the reference forwards to flash-attn's helpers when present).
"""

from __future__ import annotations

import torch

__all__ = ["index_first_axis", "pad_input", "unpad_input", "rearrange"]


def index_first_axis(tensor: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    return tensor.reshape(tensor.shape[0], -1).index_select(0, indices).reshape(-1, *tensor.shape[1:])


def unpad_input(hidden_states: torch.Tensor, attention_mask: torch.Tensor, unused_mask=None):
    """[b, s, ...] -> ([total, ...], indices, cu_seqlens int32 [b+1], max_seqlen, seqlens) over the positions where mask is 1."""
    mask = attention_mask.bool() if unused_mask is None else (attention_mask.bool() | unused_mask.bool())
    seqlens = attention_mask.sum(-1, dtype=torch.int32)
    used = mask.sum(-1, dtype=torch.int32)
    indices = torch.nonzero(mask.flatten(), as_tuple=False).flatten()
    cu = torch.nn.functional.pad(torch.cumsum(used, 0, dtype=torch.int32), (1, 0))
    flat = hidden_states.reshape(-1, *hidden_states.shape[2:])
    return index_first_axis(flat, indices), indices, cu, int(used.max()) if used.numel() else 0, seqlens


def pad_input(hidden_states: torch.Tensor, indices: torch.Tensor, batch: int, seqlen: int) -> torch.Tensor:
    out = torch.zeros(batch * seqlen, *hidden_states.shape[1:], dtype=hidden_states.dtype, device=hidden_states.device)
    out[indices] = hidden_states
    return out.view(batch, seqlen, *hidden_states.shape[1:])


def rearrange(tensor: torch.Tensor, pattern: str, **axes) -> torch.Tensor:
    from einops import rearrange as _r

    return _r(tensor, pattern, **axes)
