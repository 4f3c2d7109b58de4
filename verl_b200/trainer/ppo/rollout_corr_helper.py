"""Rollout correction: importance-sampling weights and rejection masks for rollout/training policy mismatch.

The rollout engine and the trainer may assign slightly different probabilities to the same token (different
kernels, batch shapes, quantised rollout weights).  These helpers compute truncated importance weights
``w = min(pi_train / pi_rollout, C)`` at token or sequence level and rejection masks that drop tokens /
sequences whose ratio statistics leave a trust band, plus diagnostics of the mismatch.

Parity target: ``verl/trainer/ppo/rollout_corr_helper.py`` (``compute_rollout_rejection_mask`` :197,
``compute_rollout_correction_weights`` :522, ``compute_rollout_correction_and_rejection_mask`` :786,
``compute_offpolicy_metrics`` :904, ``compute_rollout_correction_and_add_to_batch`` :1013, ``apply_bypass_mode`` :1109).
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from ...protocol import DataProto
from ...utils import torch_functional as VF

__all__ = ["compute_rollout_rejection_mask", "compute_rollout_correction_weights",
           "compute_rollout_correction_and_rejection_mask", "compute_offpolicy_metrics",
           "compute_rollout_correction_and_add_to_batch", "apply_bypass_mode"]

SAFETY_BOUND = 20.0


def _parse_band(threshold, default_upper: float = 2.0) -> tuple[float, float]:
    """'lo_hi' strings, (lo, hi) pairs or a single upper bound (lower = 1/upper)."""
    if threshold is None:
        return 1.0 / default_upper, default_upper
    if isinstance(threshold, str) and "_" in threshold:
        lo, hi = threshold.split("_")
        return float(lo), float(hi)
    if isinstance(threshold, (tuple, list)):
        return float(threshold[0]), float(threshold[1])
    hi = float(threshold)
    return (1.0 / hi if hi > 0 else 0.0), hi


def _seq_stat(x: torch.Tensor, mask: torch.Tensor, how: str) -> torch.Tensor:
    if how == "sum":
        return (x * mask).sum(-1)
    if how == "mean":
        return (x * mask).sum(-1) / mask.sum(-1).clamp(min=1)
    if how == "max":
        return x.masked_fill(mask == 0, float("-inf")).max(-1).values
    raise ValueError(how)


def compute_rollout_rejection_mask(log_ratio: torch.Tensor, response_mask: torch.Tensor, rollout_rs: str,
                                   rollout_rs_threshold=None) -> tuple[torch.Tensor, dict[str, float]]:
    """Mask (1 = keep) from a divergence statistic of ``log_ratio = log pi_train - log pi_rollout``.

    ``rollout_rs`` is ``{token|seq_sum|seq_mean|seq_max}_{k1|k2|k3}`` (``geometric`` = ``seq_mean_k1``).  k1 uses
    the ratio itself with a ``lo_hi`` band; k2 (= 0.5 log-ratio^2) and k3 (= r - 1 - log r) use an upper bound."""
    mask = response_mask.to(log_ratio.dtype)
    name = {"geometric": "seq_mean_k1", "token": "token_k1", "sequence": "seq_sum_k1"}.get(rollout_rs, rollout_rs)
    level, _, est = name.rpartition("_")
    lr = torch.clamp(log_ratio, -SAFETY_BOUND, SAFETY_BOUND)
    if est == "k1":
        stat_tok = lr
    elif est == "k2":
        stat_tok = 0.5 * lr.square()
    elif est == "k3":
        stat_tok = torch.exp(-lr) + lr - 1.0  # KL(rollout || train) estimator with r = pi_rollout / pi_train
    else:
        raise ValueError(f"unknown rejection estimator in '{rollout_rs}'")
    if level == "token":
        stat = stat_tok
    else:
        how = level.split("_")[1] if "_" in level else "sum"
        stat = _seq_stat(stat_tok, mask, how).unsqueeze(-1).expand_as(lr)
    if est == "k1":
        lo, hi = _parse_band(rollout_rs_threshold)
        keep = (torch.exp(stat) >= lo) & (torch.exp(stat) <= hi)
    else:
        ub = float(rollout_rs_threshold) if rollout_rs_threshold is not None else 0.01
        keep = stat <= ub
    keep = keep.to(mask.dtype) * mask
    metrics = {"rollout_corr/rollout_rs_masked_fraction": 1.0 - (keep.sum() / mask.sum().clamp(min=1)).item()}
    if level != "token":
        seq_keep = (keep.sum(-1) > 0) | (mask.sum(-1) == 0)
        metrics["rollout_corr/rollout_rs_seq_masked_fraction"] = 1.0 - seq_keep.float().mean().item()
    return keep, metrics


def compute_rollout_correction_weights(log_ratio: torch.Tensor, response_mask: torch.Tensor, rollout_is: str = "token",
                                       rollout_is_threshold: float = 2.0, rollout_is_batch_normalize: bool = False
                                       ) -> tuple[torch.Tensor, dict[str, float]]:
    """Truncated importance weights at token or sequence level (detached)."""
    mask = response_mask.to(log_ratio.dtype)
    if rollout_is == "token":
        lw = torch.clamp(log_ratio, -SAFETY_BOUND, SAFETY_BOUND)
    elif rollout_is == "sequence":
        lw = torch.clamp((log_ratio * mask).sum(-1, keepdim=True), -SAFETY_BOUND, SAFETY_BOUND).expand_as(log_ratio)
    elif rollout_is == "geometric":
        lw = torch.clamp(_seq_stat(log_ratio, mask, "mean").unsqueeze(-1), -SAFETY_BOUND, SAFETY_BOUND).expand_as(log_ratio)
    else:
        raise ValueError(f"Invalid rollout_is: {rollout_is}")
    w = torch.exp(lw)
    metrics = {"rollout_corr/rollout_is_mean": VF.masked_mean(w, mask).item(),
               "rollout_corr/rollout_is_max": w.masked_fill(mask == 0, 0).max().item(),
               "rollout_corr/rollout_is_truncated_fraction": VF.masked_mean((w > rollout_is_threshold).to(mask.dtype), mask).item()}
    w = torch.clamp(w, max=rollout_is_threshold) * mask
    if rollout_is_batch_normalize:
        w = w / VF.masked_mean(w, mask).clamp(min=1e-8)
    n_eff = (w * mask).sum() ** 2 / ((w * mask) ** 2).sum().clamp(min=1e-8)
    metrics["rollout_corr/rollout_is_eff_sample_size"] = (n_eff / mask.sum().clamp(min=1)).item()
    return w.detach(), metrics


def compute_offpolicy_metrics(old_log_prob: torch.Tensor, rollout_log_prob: Optional[torch.Tensor],
                              response_mask: torch.Tensor) -> dict[str, float]:
    """KL / perplexity diagnostics of the gap between the training policy and the rollout policy."""
    if rollout_log_prob is None:
        return {}
    mask = response_mask.to(old_log_prob.dtype)
    lr = old_log_prob - rollout_log_prob
    ppl_t = torch.exp(-_seq_stat(old_log_prob, mask, "mean"))
    ppl_r = torch.exp(-_seq_stat(rollout_log_prob, mask, "mean"))
    r = torch.exp(torch.clamp(lr, -SAFETY_BOUND, SAFETY_BOUND))
    return {"rollout_corr/kl": VF.masked_mean(-lr, mask).item(),
            "rollout_corr/k3_kl": VF.masked_mean(r - 1 - lr, mask).item(),
            "rollout_corr/training_ppl": ppl_t.mean().item(), "rollout_corr/rollout_ppl": ppl_r.mean().item(),
            "rollout_corr/log_ppl_diff": (torch.log(ppl_r) - torch.log(ppl_t)).mean().item(),
            "rollout_corr/ppl_ratio": (ppl_t / ppl_r).mean().item(),
            "rollout_corr/chi2_token": VF.masked_mean(r.square(), mask).item() - 1.0}


def compute_rollout_correction_and_rejection_mask(old_log_prob: torch.Tensor, rollout_log_prob: torch.Tensor,
                                                  response_mask: torch.Tensor, rollout_is: Optional[str] = None,
                                                  rollout_is_threshold: float = 2.0,
                                                  rollout_is_batch_normalize: bool = False,
                                                  rollout_rs: Optional[str] = None, rollout_rs_threshold=None
                                                  ) -> tuple[Optional[DataProto], torch.Tensor, dict[str, float]]:
    """Returns (DataProto{'rollout_is_weights'} or None, modified response mask, metrics)."""
    lr = (old_log_prob - rollout_log_prob).detach()
    metrics = compute_offpolicy_metrics(old_log_prob.detach(), rollout_log_prob, response_mask)
    new_mask = response_mask
    if rollout_rs:
        keep, m = compute_rollout_rejection_mask(lr, response_mask, rollout_rs, rollout_rs_threshold)
        new_mask = keep.to(response_mask.dtype)
        metrics.update(m)
    proto = None
    if rollout_is:
        w, m = compute_rollout_correction_weights(lr, response_mask, rollout_is, rollout_is_threshold, rollout_is_batch_normalize)
        proto = DataProto.from_dict(tensors={"rollout_is_weights": w})
        metrics.update(m)
    return proto, new_mask, metrics


def compute_rollout_correction_and_add_to_batch(batch: DataProto, rollout_corr_config) -> tuple[DataProto, dict]:
    g = rollout_corr_config.get
    proto, new_mask, metrics = compute_rollout_correction_and_rejection_mask(
        old_log_prob=batch.batch["old_log_probs"], rollout_log_prob=batch.batch["rollout_log_probs"],
        response_mask=batch.batch["response_mask"], rollout_is=g("rollout_is"), rollout_is_threshold=g("rollout_is_threshold", 2.0),
        rollout_is_batch_normalize=g("rollout_is_batch_normalize", False), rollout_rs=g("rollout_rs"),
        rollout_rs_threshold=g("rollout_rs_threshold"))
    if proto is not None:
        batch = batch.union(proto)
    batch.batch["response_mask"] = new_mask
    return batch, metrics


def apply_bypass_mode(batch: DataProto, rollout_corr_config=None, policy_loss_config=None) -> None:
    """Use the rollout log-probs as the old log-probs (skips the old-policy forward pass) and route the actor
    through the ``bypass_mode`` policy loss."""
    assert "rollout_log_probs" in batch.batch.keys(), "bypass mode needs rollout_log_probs from the rollout engine"
    batch.batch["old_log_probs"] = batch.batch["rollout_log_probs"]
    if policy_loss_config is not None:
        policy_loss_config["loss_mode"] = "bypass_mode"
        policy_loss_config["rollout_correction"] = rollout_corr_config
