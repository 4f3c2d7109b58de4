"""Data carriers and metric aggregation of the fully-asynchronous pipeline.

Parity target: ``verl/experimental/fully_async_policy/detach_utils.py`` (``RolloutSample``, ``MetricsAggregator``,
``assemble_batch_from_rollout_samples``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np

__all__ = ["RolloutSample", "MetricsAggregator"]


@dataclass
class RolloutSample:
    """One prompt with its ``n`` finished trajectories, as it travels through the message queue."""

    sample_id: str
    uid: str
    trajectories: list  # AgentLoopOutput objects
    prompt: dict = field(default_factory=dict)
    param_version_start: int = 0
    param_version_end: int = 0
    processing_time: float = 0.0
    failed: bool = False

    @property
    def staleness_span(self) -> int:
        return self.param_version_end - self.param_version_start


class MetricsAggregator:
    """Accumulates per-step metric dictionaries between two weight synchronisations and reduces them by name:
    ``*/max`` -> max, ``*/min`` -> min, ``timing_s/*`` and counters (``*/count``, ``*_total``) -> sum, everything else
    -> mean weighted by the number of samples of the step."""

    def __init__(self):
        self.rows: list[tuple[dict, int]] = []

    def add_step_metrics(self, metrics: dict, sample_count: int = 1) -> None:
        self.rows.append(({k: float(v) for k, v in metrics.items() if isinstance(v, (int, float, np.floating, np.integer))}, int(sample_count)))

    def get_aggregated_metrics(self) -> dict[str, float]:
        out: dict[str, float] = {}
        keys = sorted({k for m, _ in self.rows for k in m})
        for k in keys:
            vals = [(m[k], w) for m, w in self.rows if k in m]
            leaf = k.split("/")[-1]
            if leaf == "max":
                out[k] = max(v for v, _ in vals)
            elif leaf == "min":
                out[k] = min(v for v, _ in vals)
            elif k.startswith("timing_s/") or leaf == "count" or leaf.endswith("_total"):
                out[k] = sum(v for v, _ in vals)
            else:
                tw = sum(w for _, w in vals)
                out[k] = sum(v * w for v, w in vals) / max(1, tw)
        return out

    def reset(self) -> None:
        self.rows = []
