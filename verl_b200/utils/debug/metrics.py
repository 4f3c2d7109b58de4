"""Diagnostics comparing the rollout engine's token log-probs with the trainer's recomputation on the same tokens.

Parity target: ``verl/utils/debug/metrics.py`` (``calculate_token_list_diff`` :23, ``pearson_correlation_coefficient`` :48,
``calculate_log_prob_diff`` :58, ``calculate_debug_metrics`` :63).
"""

from __future__ import annotations

import torch

__all__ = ["calculate_token_list_diff", "pearson_correlation_coefficient", "calculate_log_prob_diff", "calculate_debug_metrics"]


def calculate_token_list_diff(tensor1: torch.Tensor, tensor2: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Per row: fraction of valid positions where the two token tensors differ."""
    if tensor1.numel() == 0 or tensor2.numel() == 0:
        return torch.zeros(tensor1.shape[0], dtype=torch.float32, device=tensor1.device)
    m = mask.bool()
    diff = ((tensor1 != tensor2) & m).sum(-1).float()
    return diff / m.sum(-1).clamp(min=1).float()


def pearson_correlation_coefficient(tensor1: torch.Tensor, tensor2: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    m = mask.bool()
    a, b = tensor1[m].double(), tensor2[m].double()
    if a.numel() < 2:
        return torch.tensor(float("nan"))
    a, b = a - a.mean(), b - b.mean()
    return ((a * b).sum() / (a.norm() * b.norm()).clamp(min=1e-30)).float()


def calculate_log_prob_diff(log_probs1: torch.Tensor, log_probs2: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """|p1 - p2| in probability space at the valid positions (flat)."""
    return (log_probs1.exp() - log_probs2.exp()).abs()[mask.bool()]


def calculate_debug_metrics(data) -> dict:
    """``data.batch`` holds ``rollout_log_probs``, ``old_log_probs`` and a response mask: how well do the two agree?"""
    b = data.batch
    roll, old = b["rollout_log_probs"].float(), b["old_log_probs"].float()
    if "response_mask" in b:
        mask = b["response_mask"]
    else:
        R = b["responses"].size(1)
        mask = b["attention_mask"][:, -R:]
    d = calculate_log_prob_diff(roll, old, mask)
    valid = mask.bool()
    return {
        "training/rollout_probs_diff_valid": int(valid.any()),
        "training/rollout_probs_diff_max": d.max().item() if d.numel() else 0.0,
        "training/rollout_probs_diff_mean": d.mean().item() if d.numel() else 0.0,
        "training/rollout_probs_diff_std": d.std().item() if d.numel() > 1 else 0.0,
        "training/rollout_actor_probs_pearson_corr": float(pearson_correlation_coefficient(roll.exp(), old.exp(), mask)),
    }
