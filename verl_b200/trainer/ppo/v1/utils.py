"""Helpers of the replay-buffer trainers.

``compute_advantage_for_multi_trajectories``: an agent-loop session may hand back several training rows (a long session cut
into pieces by context compaction, a multi-agent episode with one row per agent, ...). They are stored as
``{uid}_{session}_{index}``; only the LAST row of a session carries the session's outcome. For the group-relative estimator
the advantage is therefore computed over the final rows alone (one per session, grouped by prompt) and every other row of the
session receives its session's value on its own response tokens. Estimators that work token by token (GAE and the rest) see
the batch unchanged.

Parity target: ``verl/trainer/ppo/v1/utils.py:148-217``.
"""

from __future__ import annotations

from typing import Any, Optional, Sequence

import torch

from ..core_algos import AdvantageEstimator
from ..ray_trainer import compute_advantage

__all__ = ["split_trajectory_key", "has_multi_trajectory_sessions", "compute_advantage_for_multi_trajectories", "StepMetricsAggregator"]


def split_trajectory_key(key: str) -> tuple[str, str, int]:
    """``{uid}_{session}_{index}`` -> (uid, session, index); the uid may itself contain underscores."""
    parts = str(key).rsplit("_", 2)
    if len(parts) != 3:
        raise ValueError(f"Unexpected key format: {key}")
    return parts[0], parts[1], int(parts[2])


def has_multi_trajectory_sessions(batch_keys: Sequence[str]) -> bool:
    seen = set()
    for k in batch_keys:
        uid, session, _ = split_trajectory_key(k)
        if (uid, session) in seen:
            return True
        seen.add((uid, session))
    return False


def compute_advantage_for_multi_trajectories(data, batch_keys: Sequence[str], adv_estimator, gamma: float = 1.0, lam: float = 1.0,
                                             num_repeat: int = 1, norm_adv_by_std_in_grpo: bool = True, config: Any = None,
                                             dp: Optional[Any] = None):
    kw = dict(adv_estimator=adv_estimator, gamma=gamma, lam=lam, num_repeat=num_repeat,
              norm_adv_by_std_in_grpo=norm_adv_by_std_in_grpo, config=config)
    if dp is not None:
        kw["dp"] = dp
    if str(adv_estimator) not in ("grpo", str(AdvantageEstimator.GRPO)) and adv_estimator != AdvantageEstimator.GRPO:
        return compute_advantage(data, **kw)
    assert len(batch_keys) == len(data), (len(batch_keys), len(data))
    final_row: dict[tuple[str, str], tuple[int, int]] = {}   # session -> (highest index seen, its row)
    session_of_row = []
    for row, key in enumerate(batch_keys):
        uid, session, index = split_trajectory_key(key)
        session_of_row.append((uid, session))
        if (uid, session) not in final_row or final_row[(uid, session)][0] < index:
            final_row[(uid, session)] = (index, row)
    finals = [row for _, row in final_row.values()]
    slot = {s: i for i, s in enumerate(final_row)}
    scored = compute_advantage(data.select_idxs(finals), **kw)
    # the group-relative advantage is one number per sequence, spread over its response tokens: read it at the first of them
    first = scored.batch["response_mask"].argmax(dim=1)
    per_session = scored.batch["advantages"][torch.arange(len(scored)), first]
    idx = torch.tensor([slot[s] for s in session_of_row], device=per_session.device)
    adv = per_session[idx].unsqueeze(-1) * data.batch["response_mask"].to(per_session.dtype)
    data.batch["advantages"] = adv
    data.batch["returns"] = adv.clone()
    return data


class StepMetricsAggregator:
    """Reduces the metric dictionaries of the optimizer rounds of ONE trainer step (``parameter_sync_step`` rounds between
    two weight hand-overs) to the step's record.

    By name, first match: the eviction counters of the replay buffer are summed, ``training/global_step`` and learning
    rates keep their last value, ``timing_s/*`` and ``timing_per_token_ms/*`` are summed, names with max / min / sum|total
    reduce accordingly, everything else is a mean weighted by the number of samples of each round (the staleness mean of
    evicted samples is weighted by how many were evicted in that round). Dictionary-valued metrics (reward histograms of
    filtered groups) are merged by adding their counts. ``global_seqlen/minmax_diff`` is recomputed from the reduced max and
    min.

    Parity target: ``verl/trainer/ppo/v1/utils.py:26-146``."""

    SUM = tuple(f"{p}/{k}/{s}" for p in ("training", "validation")
                for k, s in (("off_policy", "evicted_samples"), ("filter_groups", "evicted_samples"),
                             ("filter_groups", "discarded_surplus_samples"), ("rollout_failure", "evicted_samples")))
    LAST = ("training/global_step", "training/rollout_probs_diff_valid")

    def __init__(self):
        self.reset()

    def reset(self) -> None:
        self.values: dict[str, list[float]] = {}
        self.weights: dict[str, list[int]] = {}
        self.counts: dict[str, dict] = {}
        self.step_count = 0

    @classmethod
    def rule(cls, name: str) -> str:
        if name in cls.SUM:
            return "sum"
        if name in cls.LAST:
            return "last"
        low = name.lower()
        if low == "lr" or low.endswith(("/lr", "_lr")):
            return "last"
        if "timing_s/" in low or "timing_per_token_ms/" in low:
            return "sum"
        for words, how in ((("max",), "max"), (("min",), "min"), (("sum", "total"), "sum")):
            if any(w in low for w in words):
                return how
        return "weighted"

    @staticmethod
    def _weight(name: str, metrics: dict, sample_count: int) -> int:
        if name.endswith("/off_policy/evicted_samples_staleness/mean"):
            n = metrics.get(name.rsplit("_staleness/mean", 1)[0], sample_count)
            n = n.item() if hasattr(n, "item") else n
            if isinstance(n, (int, float)):
                return int(n)
        return int(sample_count)

    def add_step_metrics(self, metrics: dict, sample_count: int = 0) -> None:
        self.step_count += 1
        for k, v in metrics.items():
            if isinstance(v, bool):
                continue
            if isinstance(v, dict):
                acc = self.counts.setdefault(k, {})
                for kk, n in v.items():
                    acc[kk] = acc.get(kk, 0) + n
                continue
            if hasattr(v, "item") and getattr(v, "numel", lambda: 2)() == 1:
                v = v.item()
            if isinstance(v, (int, float)) or type(v).__module__ == "numpy" and getattr(v, "ndim", 1) == 0:
                self.values.setdefault(k, []).append(float(v))
                self.weights.setdefault(k, []).append(self._weight(k, metrics, sample_count))

    def get_aggregated_metrics(self) -> dict:
        if self.step_count == 0:
            return {}
        out: dict = {}
        for k, vals in self.values.items():
            how = self.rule(k)
            if how == "last":
                out[k] = vals[-1]
            elif how == "sum":
                out[k] = float(sum(vals))
            elif how == "max":
                out[k] = max(vals)
            elif how == "min":
                out[k] = min(vals)
            else:
                w = self.weights[k]
                out[k] = sum(v * c for v, c in zip(vals, w)) / sum(w) if len(w) == len(vals) and sum(w) > 0 else sum(vals) / len(vals)
        out.update({k: dict(c) for k, c in self.counts.items() if c})
        if {"global_seqlen/minmax_diff", "global_seqlen/max", "global_seqlen/min"} <= set(out):
            out["global_seqlen/minmax_diff"] = out["global_seqlen/max"] - out["global_seqlen/min"]
        return out
