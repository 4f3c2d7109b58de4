"""Tensor helpers shared by algorithms, losses and workers.

Parity target: ``verl/utils/torch_functional.py`` (log-prob / entropy from logits :73-260, masked
statistics :273-346, response masks :349, distributed scalar statistics :940-983, LR schedules).
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

__all__ = [
    "logprobs_from_logits", "entropy_from_logits", "entropy_from_logits_with_chunking", "masked_sum", "masked_mean",
    "masked_var", "masked_whiten", "clip_by_value", "get_response_mask", "get_eos_mask", "compute_position_id_with_mask",
    "pad_sequence_to_length", "pad_2d_list_to_length", "postprocess_data", "allgather_dict_tensors",
    "broadcast_dict_tensor", "distributed_mean_max_min_std", "distributed_masked_mean",
    "get_constant_schedule_with_warmup", "get_cosine_schedule_with_warmup", "get_wsd_schedule_with_warmup",
    "logprobs_from_logits_v2", "gather_from_labels", "split_dict_tensor_into_batches", "expand_as_nested",
]


def gather_from_labels(data: torch.Tensor, label: torch.Tensor) -> torch.Tensor:
    return torch.gather(data, -1, label.unsqueeze(-1)).squeeze(-1)


def logprobs_from_logits_v2(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Row-wise ``logit[label] - logsumexp`` without materialising the full log-softmax in fp32 at once."""
    if logits.dtype in (torch.float32, torch.float64):
        picked = gather_from_labels(logits, labels)
        lse = torch.stack([torch.logsumexp(row, dim=-1) for row in logits]) if logits.dim() > 2 else torch.logsumexp(logits, -1)
        return picked - lse
    out = []
    for row_logits, row_labels in zip(logits, labels):
        lsm = F.log_softmax(row_logits.float(), dim=-1)
        out.append(gather_from_labels(lsm, row_labels))
    return torch.stack(out)


def logprobs_from_logits(logits: torch.Tensor, labels: torch.Tensor, inplace_backward: bool = True) -> torch.Tensor:
    """Log-probabilities of ``labels`` under ``softmax(logits)``; any leading shape."""
    shape = labels.shape
    flat = logits.reshape(-1, logits.shape[-1])
    lab = labels.reshape(-1)
    lp = gather_from_labels(flat.float(), lab) - torch.logsumexp(flat.float(), dim=-1)
    return lp.reshape(shape)


def entropy_from_logits(logits: torch.Tensor) -> torch.Tensor:
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    return lse - (torch.softmax(lf, dim=-1) * lf).sum(dim=-1)


def entropy_from_logits_with_chunking(logits: torch.Tensor, chunk_size: int = 2048) -> torch.Tensor:
    flat = logits.reshape(-1, logits.shape[-1])
    out = torch.empty(flat.shape[0], dtype=torch.float32, device=logits.device)
    for s in range(0, flat.shape[0], chunk_size):
        out[s : s + chunk_size] = entropy_from_logits(flat[s : s + chunk_size])
    return out.reshape(logits.shape[:-1])


# ----------------------------------------------------------------------------------------------- masked stats
def masked_sum(values: torch.Tensor, mask: torch.Tensor, axis=None) -> torch.Tensor:
    """Sum over unmasked entries; NaNs hidden behind the mask do not leak into the result."""
    safe = torch.where(mask.bool(), values, torch.zeros((), dtype=values.dtype, device=values.device))
    return (safe * mask).sum(axis) if axis is not None else (safe * mask).sum()


def masked_mean(values: torch.Tensor, mask: torch.Tensor, axis=None) -> torch.Tensor:
    denom = mask.sum(axis) if axis is not None else mask.sum()
    return masked_sum(values, mask, axis) / (denom + 1e-8)


def masked_var(values: torch.Tensor, mask: torch.Tensor, unbiased: bool = True) -> torch.Tensor:
    mean = masked_mean(values, mask)
    var = masked_mean((values - mean) ** 2, mask)
    if unbiased:
        n = mask.sum()
        if n == 0:
            raise ValueError("At least one element in the mask has to be 1.")
        if n == 1:
            raise ValueError("The sum of the mask is one, which can cause a division by zero.")
        var = var * (n / (n - 1))
    return var


def masked_whiten(values: torch.Tensor, mask: torch.Tensor, shift_mean: bool = True) -> torch.Tensor:
    mean, var = masked_mean(values, mask), masked_var(values, mask)
    out = (values - mean) * torch.rsqrt(var + 1e-8)
    return out if shift_mean else out + mean


def clip_by_value(x: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor) -> torch.Tensor:
    return torch.max(torch.min(x, hi), lo)


# ----------------------------------------------------------------------------------------------- masks / padding
def get_response_mask(response_id: torch.Tensor, eos_token=2, dtype=torch.int64) -> torch.Tensor:
    """1 up to and including the first EOS of every row, 0 afterwards."""
    eos = [eos_token] if isinstance(eos_token, int) else list(eos_token)
    is_eos = torch.isin(response_id, torch.tensor(eos, device=response_id.device))
    after = (torch.cumsum(is_eos.long(), dim=1) - is_eos.long()) > 0
    return (~after).to(dtype)


get_eos_mask = get_response_mask


def compute_position_id_with_mask(mask: torch.Tensor) -> torch.Tensor:
    return torch.clip(torch.cumsum(mask, dim=-1) - 1, min=0, max=None)


def pad_sequence_to_length(t: torch.Tensor, max_seq_len: int, pad_token_id, left_pad: bool = False) -> torch.Tensor:
    if t.shape[-1] >= max_seq_len:
        return t
    pad = (max_seq_len - t.shape[-1], 0) if left_pad else (0, max_seq_len - t.shape[-1])
    return F.pad(t, pad, "constant", pad_token_id)


def pad_2d_list_to_length(rows, pad_token_id, max_length: Optional[int] = None) -> torch.Tensor:
    n = max(len(r) for r in rows) if rows else 0
    n = max(n, max_length or 0)
    return torch.tensor([list(r) + [pad_token_id] * (n - len(r)) for r in rows])


def postprocess_data(input_ids, attention_mask, max_length: int, pad_token_id: int, left_pad: bool = True,
                     truncation: str = "error"):
    """Pad (left by default) or truncate a [1, L] prompt to ``max_length``."""
    L = input_ids.shape[-1]
    if L < max_length:
        input_ids = pad_sequence_to_length(input_ids, max_length, pad_token_id, left_pad)
        attention_mask = pad_sequence_to_length(attention_mask, max_length, 0, left_pad)
    elif L > max_length:
        if truncation == "left":
            input_ids, attention_mask = input_ids[:, -max_length:], attention_mask[:, -max_length:]
        elif truncation == "right":
            input_ids, attention_mask = input_ids[:, :max_length], attention_mask[:, :max_length]
        elif truncation == "middle":
            l, r = max_length // 2, max_length - max_length // 2
            input_ids = torch.cat([input_ids[:, :l], input_ids[:, -r:]], -1)
            attention_mask = torch.cat([attention_mask[:, :l], attention_mask[:, -r:]], -1)
        else:
            raise NotImplementedError(f"sequence_length={L} is larger than max_length={max_length}")
    return input_ids, attention_mask


def split_dict_tensor_into_batches(tensors, batch_size: int):
    n = next(iter(tensors.values())).shape[0]
    return [{k: v[s : s + batch_size] for k, v in tensors.items()} for s in range(0, n, batch_size)]


def expand_as_nested(t: torch.Tensor, lengths) -> list[torch.Tensor]:
    return [t[i, : int(n)] for i, n in enumerate(lengths)]


# ----------------------------------------------------------------------------------------------- collectives
def allgather_dict_tensors(tensors: dict, size: int, group=None, dim: int = 0) -> dict:
    out = {}
    for k in sorted(tensors.keys()):
        v = tensors[k]
        parts = [torch.empty_like(v) for _ in range(size)]
        dist.all_gather(parts, v, group=group)
        out[k] = torch.cat(parts, dim=dim)
    return out


def broadcast_dict_tensor(tensors: dict, src: int, group=None) -> None:
    for k in sorted(tensors.keys()):
        dist.broadcast(tensors[k], src=src, group=group)


def distributed_mean_max_min_std(local: torch.Tensor, compute_max=True, compute_min=True, compute_std=True):
    n = torch.tensor(float(local.numel()), device=local.device)
    s = local.float().sum()
    if dist.is_initialized():
        dist.all_reduce(n)
        dist.all_reduce(s)
    mean = s / n
    mx = mn = sd = None
    if compute_max:
        mx = local.max().float()
        if dist.is_initialized():
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    if compute_min:
        mn = local.min().float()
        if dist.is_initialized():
            dist.all_reduce(mn, op=dist.ReduceOp.MIN)
    if compute_std:
        sq = ((local.float() - mean) ** 2).sum()
        if dist.is_initialized():
            dist.all_reduce(sq)
        sd = torch.sqrt(sq / (n - 1).clamp(min=1))
    return mean, mx, mn, sd


def distributed_masked_mean(local: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    num = (local * mask).sum().float()
    den = mask.sum().float()
    if dist.is_initialized():
        dist.all_reduce(num)
        dist.all_reduce(den)
    return num / den


# ----------------------------------------------------------------------------------------------- LR schedules
def get_constant_schedule_with_warmup(optimizer, num_warmup_steps: int, last_epoch: int = -1):
    from torch.optim.lr_scheduler import LambdaLR

    return LambdaLR(optimizer, lambda s: min(1.0, float(s) / float(max(1, num_warmup_steps))) if num_warmup_steps > 0 else 1.0,
                    last_epoch)


def cosine_factor(step: int, warmup: int, total: int, min_ratio: float = 0.0, cycles: float = 0.5,
                  init_ratio: float = 0.0) -> float:
    if step < warmup:
        return init_ratio + (1.0 - init_ratio) * step / max(1, warmup)
    prog = (step - warmup) / max(1, total - warmup)
    return min_ratio + (1 - min_ratio) * max(0.0, 0.5 * (1.0 + math.cos(math.pi * cycles * 2.0 * prog)))


def get_cosine_schedule_with_warmup(optimizer, num_warmup_steps: int, num_training_steps: int, min_lr_ratio: float = 0.0,
                                    num_cycles: float = 0.5, last_epoch: int = -1, init_lr_ratio: float = 0.0):
    from torch.optim.lr_scheduler import LambdaLR

    return LambdaLR(optimizer, lambda s: cosine_factor(s, num_warmup_steps, num_training_steps, min_lr_ratio,
                                                       num_cycles, init_lr_ratio), last_epoch)


def wsd_factor(step: int, warmup: int, total: int, stable_ratio: float = 0.9, min_ratio: float = 0.0) -> float:
    if step < warmup:
        return step / max(1, warmup)
    stable_end = warmup + int((total - warmup) * stable_ratio)
    if step < stable_end:
        return 1.0
    prog = (step - stable_end) / max(1, total - stable_end)
    return max(min_ratio, 1.0 - (1.0 - min_ratio) * prog)


def get_wsd_schedule_with_warmup(optimizer, num_warmup_steps: int, num_training_steps: int, min_lr_ratio: float = 0.0,
                                 stable_ratio: float = 0.9, last_epoch: int = -1):
    from torch.optim.lr_scheduler import LambdaLR

    return LambdaLR(optimizer, lambda s: wsd_factor(s, num_warmup_steps, num_training_steps, stable_ratio, min_lr_ratio),
                    last_epoch)
