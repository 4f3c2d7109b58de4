"""Rollout correction: importance-sampling weights and rejection masks for rollout/training policy mismatch.

The rollout engine and the trainer may assign slightly different probabilities to the same token (different
kernels, batch shapes, quantised rollout weights, stale weights in the asynchronous trainers). These helpers compute
importance weights ``pi_train / pi_rollout`` at token or sequence level (truncated, or zeroed outside a band), rejection
masks that drop tokens / sequences whose divergence statistics leave a trust region, and diagnostics of the mismatch.

With ``d = log pi_train - log pi_rollout`` per token, the three divergence estimators are ``k1 = -d``,
``k2 = d^2 / 2`` and ``k3 = exp(d) - 1 - d``; a rejection option is ``<level>_<estimator>`` with level ``token``,
``seq_sum``, ``seq_mean`` or ``seq_max`` (``seq_max`` only for k2 / k3). k1 options are banded in ratio space
(``"lower_upper"``, or a single upper bound u meaning [1/u, u]); k2 / k3 options take one upper bound. Several options,
comma separated, must all pass.

Parity target: ``verl/trainer/ppo/rollout_corr_helper.py`` (``compute_rollout_rejection_mask`` :197,
``compute_rs_metrics`` :416, ``compute_rollout_correction_weights`` :522, ``compute_is_metrics`` :660,
``compute_rollout_correction_and_rejection_mask`` :786, ``compute_offpolicy_metrics`` :904,
``compute_rollout_correction_and_add_to_batch`` :1013, ``compute_rollout_corr_metrics_from_logprobs`` :1070,
``apply_bypass_mode`` :1109).
"""

from __future__ import annotations

import math
from typing import Any, Optional

import torch

from ...protocol import DataProto
from ...utils import torch_functional as VF

__all__ = ["compute_rollout_rejection_mask", "compute_rs_metrics", "compute_rollout_correction_weights", "compute_is_metrics",
           "compute_rollout_correction_and_rejection_mask", "compute_offpolicy_metrics",
           "compute_rollout_correction_and_add_to_batch", "compute_rollout_corr_metrics_from_logprobs", "apply_bypass_mode",
           "SUPPORTED_ROLLOUT_RS_OPTIONS"]

SAFETY_BOUND = 20.0
_ESTIMATORS = {"k1": lambda d: -d, "k2": lambda d: 0.5 * d * d, "k3": lambda d: torch.exp(d) - 1.0 - d}
_LEVELS = ("token", "seq_sum", "seq_mean", "seq_max")
SUPPORTED_ROLLOUT_RS_OPTIONS = frozenset(f"{lv}_{k}" for lv in _LEVELS for k in _ESTIMATORS if not (lv == "seq_max" and k == "k1"))
_ALIASES = {"geometric": "seq_mean_k1", "token": "token_k1", "sequence": "seq_sum_k1"}


def _positive(x: str, what: str) -> float:
    try:
        v = float(x)
    except ValueError as e:
        raise ValueError(f"invalid number '{x}' in {what}") from e
    if v <= 0:
        raise ValueError(f"{what}: bounds must be positive, got {x}")
    return v


def _parse_rollout_is_threshold(spec) -> tuple[float, Optional[float]]:
    """(upper, lower or None). A number (or numeric string) truncates at ``upper``; ``"lower_upper"`` zeroes weights
    outside the band."""
    if isinstance(spec, bool) or not isinstance(spec, (int, float, str)):
        raise TypeError("rollout_is_threshold must be a number or a 'lower_upper' string")
    if isinstance(spec, (int, float)):
        upper, lower = float(spec), None
        if upper <= 0:
            raise ValueError(f"rollout_is_threshold upper bound must be positive, got {upper}")
        return upper, lower
    text = spec.strip()
    if not text:
        raise ValueError("rollout_is_threshold must not be empty")
    if "_" in text:
        lo, hi = text.split("_", 1)
        lower, upper = _positive(lo, "rollout_is_threshold"), _positive(hi, "rollout_is_threshold")
        if lower > upper:
            raise ValueError("rollout_is_threshold: lower bound above upper bound")
        return upper, lower
    return _positive(text, "rollout_is_threshold"), None


def _parse_rollout_rs_thresholds(options: list[str], spec) -> dict[str, tuple[Optional[float], float]]:
    """option -> (lower or None, upper). One entry for all options or one per option, comma separated."""
    if spec is None:
        raise ValueError("rollout_rs_threshold must be provided for rejection sampling")
    if isinstance(spec, bool) or not isinstance(spec, (int, float, str)):
        raise TypeError("rollout_rs_threshold must be a string or a number")
    parts = [str(spec)] if isinstance(spec, (int, float)) else [p.strip() for p in spec.split(",") if p.strip()]
    if not parts or len(parts) not in (1, len(options)):
        raise ValueError(f"rollout_rs_threshold needs one entry, or one per option ({len(options)}), got {len(parts)}")
    if len(parts) == 1:
        parts = parts * len(options)
    out: dict[str, tuple[Optional[float], float]] = {}
    for opt, text in zip(options, parts):
        what = f"rollout_rs_threshold of '{opt}'"
        if opt.endswith("k1"):
            if "_" in text:
                lo, hi = text.split("_", 1)
                lower, upper = _positive(lo, what), _positive(hi, what)
            else:
                upper = _positive(text, what)
                lower = 1.0 / upper
            if lower > upper:
                raise ValueError(f"{what}: lower bound above upper bound")
            out[opt] = (lower, upper)
        else:
            if "_" in text:
                raise ValueError(f"{what}: a single upper bound without '_' is expected")
            out[opt] = (None, _positive(text, what))
    return out


def _per_sequence(values: torch.Tensor, mask: torch.Tensor, how: str) -> torch.Tensor:
    if how == "sum":
        return VF.masked_sum(values, mask, axis=-1)
    if how == "mean":
        return VF.masked_mean(values, mask, axis=-1)
    top = values.masked_fill(~mask.bool(), float("-inf")).max(dim=-1).values
    return torch.where(torch.isinf(top) & (top < 0), torch.zeros_like(top), top)   # a sequence without tokens: 0


def compute_rs_metrics(option_name: str, rs_statistic: torch.Tensor, response_mask: torch.Tensor, seq_valid_mask: torch.Tensor, *,
                       level: str, per_sequence_values: Optional[torch.Tensor], rollout_rs_threshold: float,
                       rollout_rs_threshold_lower: float, apply_lower_threshold: bool) -> dict[str, float]:
    """Statistics of one rejection option's statistic (per token, already broadcast for sequence levels) against its
    bounds: mean / max / min / std, fractions beyond the bounds, and the same per sequence."""
    if not response_mask.any():
        raise ValueError("response_mask must contain at least one valid token")
    pre = f"rollout_rs_{option_name}"
    valid = response_mask.bool()
    seq = per_sequence_values if per_sequence_values is not None else VF.masked_mean(rs_statistic, response_mask, axis=-1)
    seq = seq.reshape(seq.shape[0], -1)[:, 0][seq_valid_mask]
    hi, lo = rollout_rs_threshold, rollout_rs_threshold_lower
    m: dict[str, float] = {f"{pre}_mean": VF.masked_mean(rs_statistic, response_mask).item()}
    by_seq = level == "sequence" and seq.numel() > 0
    if by_seq:
        m[f"{pre}_max"], m[f"{pre}_min"] = seq.max().item(), seq.min().item()
        m[f"{pre}_fraction_high"] = (seq > hi).float().mean().item()
        m[f"{pre}_fraction_low"] = (seq < lo).float().mean().item() if apply_lower_threshold else 0.0
    else:
        m[f"{pre}_max"] = rs_statistic.masked_fill(~valid, float("-inf")).max().item()
        m[f"{pre}_min"] = rs_statistic.masked_fill(~valid, float("inf")).min().item()
        m[f"{pre}_fraction_high"] = VF.masked_mean((rs_statistic > hi).float(), response_mask).item()
        m[f"{pre}_fraction_low"] = VF.masked_mean((rs_statistic < lo).float(), response_mask).item() if apply_lower_threshold else 0.0
    if response_mask.sum() > 1:  # spread of the statistic inside its bounds
        inside = rs_statistic.clamp(min=lo if apply_lower_threshold else 0.0, max=hi)
        var = VF.masked_mean(inside.square(), response_mask) - VF.masked_mean(inside, response_mask).square()
        m[f"{pre}_std"] = torch.sqrt(var.clamp(min=0.0)).item()
    else:
        m[f"{pre}_std"] = 0.0
    if seq.numel() > 0:
        m[f"{pre}_seq_mean"] = seq.mean().item()
        m[f"{pre}_seq_std"] = seq.std().item() if seq.numel() > 1 else 0.0
        m[f"{pre}_seq_max"], m[f"{pre}_seq_min"] = seq.max().item(), seq.min().item()
        m[f"{pre}_seq_max_deviation"] = seq.abs().max().item()
        m[f"{pre}_seq_fraction_high"] = (seq > hi).float().mean().item()
        if apply_lower_threshold:
            m[f"{pre}_seq_fraction_low"] = (seq < lo).float().mean().item()
    else:
        for k in ("seq_mean", "seq_std", "seq_max", "seq_min", "seq_max_deviation", "seq_fraction_high", "seq_fraction_low"):
            m[f"{pre}_{k}"] = 0.0
    return m


def compute_rollout_rejection_mask(log_ratio: torch.Tensor, response_mask: torch.Tensor, rollout_rs: str = "token_k1",
                                   rollout_rs_threshold=None) -> tuple[torch.Tensor, dict[str, float]]:
    """Hard trust region: the response mask with every token (or whole sequence) zeroed whose divergence statistic leaves
    the bounds of any requested option, and per-option metrics (keys ``rollout_rs_*``, no prefix)."""
    if not isinstance(rollout_rs, str) or not rollout_rs:
        raise ValueError("rollout_rs must be a non-empty string (comma separated for several options)")
    if rollout_rs_threshold is None:
        raise ValueError("rollout_rs_threshold must be provided for rejection sampling")
    if log_ratio.shape[0] == 0:
        return response_mask, {}
    options: list[str] = []
    for raw in rollout_rs.split(","):
        opt = _ALIASES.get(raw.strip(), raw.strip())
        if not opt:
            continue
        if opt not in SUPPORTED_ROLLOUT_RS_OPTIONS:
            raise ValueError(f"Invalid rollout_rs option: {opt}. Must be one of {sorted(SUPPORTED_ROLLOUT_RS_OPTIONS)}.")
        if opt not in options:
            options.append(opt)
    if not options:
        raise ValueError("rollout_rs must contain at least one option")
    bounds = _parse_rollout_rs_thresholds(options, rollout_rs_threshold)
    d = torch.clamp(log_ratio, min=-SAFETY_BOUND, max=SAFETY_BOUND)
    valid = response_mask.bool()
    seq_valid = response_mask.sum(dim=-1) > 0
    keep_all = torch.ones_like(response_mask, dtype=log_ratio.dtype)
    metrics: dict[str, float] = {}
    for opt in options:
        level, est = opt.rsplit("_", 1)
        tok = _ESTIMATORS[est](d)
        lower, upper = bounds[opt]
        # k1 is compared in log space against the ratio band; k2 / k3 against their upper bound
        hi = math.log(upper) if est == "k1" else upper
        lo = math.log(lower) if est == "k1" else 0.0
        if level == "token":
            stat, seq_stat = tok, None
        else:
            seq_stat = _per_sequence(tok, response_mask, level.split("_", 1)[1])
            stat = seq_stat.unsqueeze(-1).expand_as(response_mask)
        keep = (stat <= hi) & (stat >= lo) if est == "k1" else (stat <= hi)
        keep_all = keep_all * keep.to(log_ratio.dtype)
        metrics.update(compute_rs_metrics(opt, stat, response_mask, seq_valid, level="token" if level == "token" else "sequence",
                                          per_sequence_values=seq_stat, rollout_rs_threshold=hi, rollout_rs_threshold_lower=lo,
                                          apply_lower_threshold=est == "k1"))
        metrics[f"rollout_rs_{opt}_masked_fraction"] = VF.masked_mean(1 - keep.to(log_ratio.dtype), response_mask).item()
        dropped = ((~keep) & valid).any(dim=-1).to(log_ratio.dtype) * seq_valid.to(log_ratio.dtype)
        metrics[f"rollout_rs_{opt}_seq_masked_fraction"] = (dropped.sum() / seq_valid.sum()).item() if seq_valid.any() else 0.0
    metrics["rollout_rs_masked_fraction"] = VF.masked_mean(1 - keep_all, response_mask).item()
    metrics["rollout_rs_seq_masked_fraction"] = (((keep_all < 0.5) & valid).any(dim=-1)).float().mean().item()
    return (response_mask * keep_all).to(response_mask.dtype), metrics


def compute_is_metrics(rollout_is_weights: torch.Tensor, raw_rollout_is_weights: torch.Tensor, log_ratio_for_metrics: torch.Tensor,
                       response_mask: torch.Tensor, rollout_is: str, rollout_is_threshold: float,
                       rollout_is_threshold_lower: Optional[float] = None) -> dict[str, float]:
    """Statistics of the applied weights, with the raw (unprocessed) weights telling how often the bounds were hit."""
    if not response_mask.any():
        raise ValueError("response_mask must contain at least one valid token")
    hi = float(rollout_is_threshold)
    lo = 1.0 / hi if rollout_is_threshold_lower is None else float(rollout_is_threshold_lower)
    valid = response_mask.bool()
    m: dict[str, float] = {"rollout_is_mean": VF.masked_mean(rollout_is_weights, response_mask).item()}
    if rollout_is == "sequence":
        m["rollout_is_max"] = torch.exp(log_ratio_for_metrics.max().clamp(max=SAFETY_BOUND)).item()
        m["rollout_is_min"] = torch.exp(log_ratio_for_metrics.min()).item()
        m["rollout_is_ratio_fraction_high"] = (log_ratio_for_metrics > math.log(hi)).float().mean().item()
        m["rollout_is_ratio_fraction_low"] = (log_ratio_for_metrics < math.log(lo)).float().mean().item()
    else:
        m["rollout_is_max"] = rollout_is_weights.masked_fill(~valid, float("-inf")).max().item()
        m["rollout_is_min"] = rollout_is_weights.masked_fill(~valid, float("inf")).min().item()
        m["rollout_is_ratio_fraction_high"] = VF.masked_mean((raw_rollout_is_weights > hi).float(), response_mask).item()
        m["rollout_is_ratio_fraction_low"] = VF.masked_mean((raw_rollout_is_weights < lo).float(), response_mask).item()
    inside = rollout_is_weights.clamp(min=0.0, max=hi)
    mean_in = VF.masked_mean(inside, response_mask)
    if response_mask.sum() > 1:
        m["rollout_is_std"] = torch.sqrt((VF.masked_mean(inside.square(), response_mask) - mean_in.square()).clamp(min=0.0)).item()
    else:
        m["rollout_is_std"] = 0.0
    m["rollout_is_eff_sample_size"] = 1.0 / VF.masked_mean((inside / (mean_in + 1e-8)).square(), response_mask).item()
    if rollout_is_weights.dim() > 1:
        seq = VF.masked_mean(rollout_is_weights, response_mask, axis=-1)
        raw_seq = VF.masked_mean(raw_rollout_is_weights, response_mask, axis=-1)
        m["rollout_is_seq_mean"] = seq.mean().item()
        m["rollout_is_seq_std"] = seq.std().item() if seq.numel() > 1 else 0.0
        m["rollout_is_seq_max"], m["rollout_is_seq_min"] = seq.max().item(), seq.min().item()
        m["rollout_is_seq_max_deviation"] = (seq - 1.0).abs().max().item()
        m["rollout_is_seq_fraction_high"] = (raw_seq > hi).float().mean().item()
        m["rollout_is_seq_fraction_low"] = (raw_seq < lo).float().mean().item()
    return m


def compute_rollout_correction_weights(log_ratio: torch.Tensor, response_mask: torch.Tensor, rollout_is: str = "token",
                                       rollout_is_threshold=2.0, rollout_is_batch_normalize: bool = False
                                       ) -> tuple[torch.Tensor, dict[str, float]]:
    """Importance weights ``pi_train / pi_rollout`` per token or per sequence (product over the tokens), detached. A single
    threshold truncates them from above; a ``"lower_upper"`` band zeroes the weights outside it. Optionally rescaled to mean
    1 over the batch (over all data-parallel ranks when a process group is up). Metrics carry no prefix."""
    if rollout_is not in ("token", "sequence"):
        raise ValueError(f"Invalid rollout_is: {rollout_is}. Must be one of ['sequence', 'token'].")
    upper, lower = _parse_rollout_is_threshold(rollout_is_threshold)
    mask_f = response_mask.to(log_ratio.dtype)
    if rollout_is == "token":
        for_metrics = log_ratio
        raw = torch.exp(torch.clamp(log_ratio, min=-SAFETY_BOUND, max=SAFETY_BOUND))
    else:
        for_metrics = VF.masked_sum(log_ratio, response_mask, axis=-1).unsqueeze(-1)
        raw = torch.exp(torch.clamp(for_metrics, min=-SAFETY_BOUND, max=SAFETY_BOUND)).expand_as(log_ratio)
    raw = raw * mask_f
    if lower is None:
        w = raw.clamp(max=upper)
    else:
        w = torch.where((raw >= lower) & (raw <= upper), raw, torch.zeros_like(raw))
    metrics = compute_is_metrics(w, raw, for_metrics, response_mask, rollout_is, upper, lower)
    if lower is not None:
        metrics["rollout_is_oob_ratio"] = VF.masked_mean(((raw < lower) | (raw > upper)).float(), response_mask).item()
    w = w.detach()
    if rollout_is_batch_normalize:
        if rollout_is == "token":
            vals, wts = w, mask_f
        else:
            vals, wts = VF.masked_mean(w, response_mask, axis=-1), (response_mask.sum(dim=-1) > 0).to(w.dtype)
        mean = _global_masked_mean(vals, wts)
        if mean > 1e-8:
            w = w / mean
            metrics["rollout_is_batch_norm_factor"] = float(mean)
        else:
            metrics["rollout_is_batch_norm_factor"] = 1.0
    return w, metrics


def _global_masked_mean(values: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """Mean of ``values`` weighted by ``weights`` over every rank of the default process group (local when none is up)."""
    acc = torch.stack([(values * weights).sum(), weights.sum()]).to(torch.float64)
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.all_reduce(acc)
    return (acc[0] / acc[1].clamp(min=1e-8)).to(values.dtype)


def compute_offpolicy_metrics(old_log_prob: torch.Tensor, rollout_log_prob: Optional[torch.Tensor],
                              response_mask: torch.Tensor) -> dict[str, Any]:
    """Gap between the training policy and the rollout policy on the sampled tokens: KL estimators, perplexities and
    chi-square divergences (keys without prefix)."""
    assert response_mask.any(), "Expected at least one valid token in response_mask"
    lp_train = VF.masked_mean(old_log_prob, response_mask, axis=-1)
    m: dict[str, Any] = {"training_ppl": torch.exp(-lp_train).mean().item(), "training_log_ppl": (-lp_train).mean().item()}
    if rollout_log_prob is None:
        return m
    d = (old_log_prob - rollout_log_prob).detach()
    lp_roll = VF.masked_mean(rollout_log_prob, response_mask, axis=-1)
    gap = lp_roll - lp_train
    d_safe = torch.clamp(d, min=-SAFETY_BOUND, max=SAFETY_BOUND)
    d_seq = torch.clamp(VF.masked_sum(d, response_mask, axis=-1), min=-SAFETY_BOUND, max=SAFETY_BOUND)
    m.update({
        "kl": VF.masked_mean(-d, response_mask).item(),
        "k3_kl": VF.masked_mean(torch.exp(d) - d - 1, response_mask).item(),
        "rollout_ppl": torch.exp(-lp_roll).mean().item(), "rollout_log_ppl": (-lp_roll).mean().item(),
        "log_ppl_diff": gap.mean().item(), "log_ppl_abs_diff": gap.abs().mean().item(),
        "log_ppl_diff_max": gap.max().item(), "log_ppl_diff_min": gap.min().item(),
        "ppl_ratio": torch.exp(gap).mean().item(),
        "chi2_token": (VF.masked_mean(torch.exp(2.0 * d_safe), response_mask) - 1.0).item(),
        "chi2_seq": (torch.exp(2.0 * d_seq).mean() - 1.0).item(),
    })
    return m


def _prefixed(metrics: dict) -> dict[str, float]:
    return {f"rollout_corr/{k}": (v.item() if isinstance(v, torch.Tensor) else v) for k, v in metrics.items()}


def compute_rollout_correction_and_rejection_mask(old_log_prob: torch.Tensor, rollout_log_prob: torch.Tensor,
                                                  response_mask: torch.Tensor, rollout_is: Optional[str] = None,
                                                  rollout_is_threshold=2.0, rollout_is_batch_normalize: bool = False,
                                                  rollout_rs: Optional[str] = None, rollout_rs_threshold=None
                                                  ) -> tuple[Optional[DataProto], torch.Tensor, dict[str, float]]:
    """Returns (DataProto{'rollout_is_weights'} or None, response mask after rejection, metrics with the ``rollout_corr/``
    prefix). Weights and rejection are independent: either can be used alone."""
    if not response_mask.any():
        raise ValueError("response_mask must contain at least one valid token")
    if old_log_prob.shape != rollout_log_prob.shape or old_log_prob.shape != response_mask.shape:
        raise ValueError(f"shapes differ: old_log_prob {tuple(old_log_prob.shape)}, rollout_log_prob {tuple(rollout_log_prob.shape)}, "
                         f"response_mask {tuple(response_mask.shape)}")
    d = (old_log_prob - rollout_log_prob).detach()
    metrics: dict[str, Any] = {}
    weights = None
    if rollout_is is not None and rollout_is_threshold is not None:
        weights, m = compute_rollout_correction_weights(d, response_mask, rollout_is, rollout_is_threshold, rollout_is_batch_normalize)
        metrics.update(m)
    new_mask = response_mask.clone()
    if rollout_rs is not None:
        if rollout_rs_threshold is None:
            raise ValueError("rollout_rs_threshold must be explicitly provided when rollout_rs is enabled")
        new_mask, m = compute_rollout_rejection_mask(d, response_mask, rollout_rs, rollout_rs_threshold)
        metrics.update(m)
    metrics.update(compute_offpolicy_metrics(old_log_prob.detach(), rollout_log_prob, response_mask))
    proto = DataProto.from_dict(tensors={"rollout_is_weights": weights}) if weights is not None else None
    return proto, new_mask, _prefixed(metrics)


def compute_rollout_correction_and_add_to_batch(batch: DataProto, rollout_corr_config) -> tuple[DataProto, dict]:
    """The response mask of ``batch`` always takes the rejection; ``rollout_is_weights`` is added only when
    ``rollout_is`` is configured, so the diagnostics can be watched before the correction is switched on."""
    g = rollout_corr_config.get
    proto, new_mask, metrics = compute_rollout_correction_and_rejection_mask(
        old_log_prob=batch.batch["old_log_probs"], rollout_log_prob=batch.batch["rollout_log_probs"],
        response_mask=batch.batch["response_mask"], rollout_is=g("rollout_is", None), rollout_is_threshold=g("rollout_is_threshold", 2.0),
        rollout_is_batch_normalize=g("rollout_is_batch_normalize", False), rollout_rs=g("rollout_rs", None),
        rollout_rs_threshold=g("rollout_rs_threshold", None))
    batch.batch["response_mask"] = new_mask
    if proto is not None:
        batch = batch.union(proto)
    return batch, metrics


def compute_rollout_corr_metrics_from_logprobs(log_prob: torch.Tensor, rollout_log_prob: torch.Tensor,
                                               response_mask: torch.Tensor) -> dict[str, float]:
    """Off-policy diagnostics of the CURRENT policy against the rollout policy (the actor calls this on every update, so
    the gap can be followed as training moves on); keys carry the ``rollout_corr/`` prefix."""
    return _prefixed(compute_offpolicy_metrics(log_prob, rollout_log_prob, response_mask))


def apply_bypass_mode(batch: DataProto, rollout_corr_config=None, policy_loss_config=None) -> None:
    """Use the rollout log-probs as the old log-probs (skips the old-policy forward pass) and route the actor
    through the ``bypass_mode`` policy loss."""
    if "rollout_log_probs" not in batch.batch.keys():
        raise ValueError("bypass_mode=True requires rollout_log_probs in batch. "
                         "Ensure rollout worker is configured to calculate_log_probs=true.")
    batch.batch["old_log_probs"] = batch.batch["rollout_log_probs"]
    if policy_loss_config is not None:
        policy_loss_config["rollout_correction"] = rollout_corr_config
        policy_loss_config["loss_mode"] = "bypass_mode"
