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

__all__ = ["split_trajectory_key", "has_multi_trajectory_sessions", "compute_advantage_for_multi_trajectories"]


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
