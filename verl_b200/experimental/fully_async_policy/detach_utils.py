"""Data carriers and metric aggregation of the fully-asynchronous pipeline.

Parity target: ``verl/experimental/fully_async_policy/detach_utils.py`` (``RolloutSample``, ``MetricsAggregator``,
``assemble_batch_from_rollout_samples``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np

__all__ = ["RolloutSample", "MetricsAggregator", "task_exception_handler", "safe_create_task"]


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
    """Collects the metric dictionaries of the training steps between two weight synchronisations and reduces them to one.

    How a name is reduced (first match wins):

    * listed by name: counters and snapshots keep their LAST value (``fully_async/count/*``, ``training/global_step``,
      ``dynamic_resource/mq_size``); ``perf/time_per_step`` and the raw seconds behind the utilisation ratios are SUMMED;
    * ``timing_s/*`` is summed (the cycle's wall clock is the sum of its steps), except the ``tool_calls/{min,mean,max}``
      statistics, which reduce like their suffix;
    * otherwise by keyword in the name: mean / avg -> mean, max -> max, min -> min, sum / total -> sum,
      ``weighted_avg`` -> mean weighted by the number of samples of each step; anything else -> mean.

    Derived afterwards from the reduced values: ``global_seqlen/minmax_diff``, ``perf/throughput`` (total tokens / (summed
    time x GPUs)), ``fully_async/trainer/idle_ratio`` (time spent waiting for samples / step time),
    ``dynamic_resource/train_resource_utilization`` (summed compute seconds / summed allocated seconds) and, when the
    rollouter's utilisation of the same cycle is handed in, ``dynamic_resource/resource_utilization``: with ``a`` GPUs that
    switch between training and generation, ``b`` GPUs that only generate and ``x`` the share of the cycle the switching
    GPUs spent generating (``timing_s/wait_for_enough_samples / timing_s/step``),
    ``((1 - x) a U_train + (x a + b) U_rollout) / (a + b)``.

    Parity target: ``verl/experimental/fully_async_policy/detach_utils.py:179-438``."""

    LAST = ("fully_async/count/total_generated_samples", "fully_async/count/stale_samples_processed",
            "fully_async/count/stale_trajectory_processed", "fully_async/count/current_param_version",
            "fully_async/count/dropped_stale_samples", "fully_async/param_version", "training/global_step",
            "dynamic_resource/mq_size")
    SUM = ("perf/time_per_step", "dynamic_resource/train_compute_time_s", "dynamic_resource/train_allocated_time_s")
    BY_SUFFIX = {"timing_s/agent_loop/tool_calls/min": "min", "timing_s/agent_loop/tool_calls/mean": "mean",
                 "timing_s/agent_loop/tool_calls/max": "max"}

    def __init__(self, total_gpus: int = 1, hybrid_gpus: int = 0, standalone_gpus: int = 0):
        self.total_gpus, self.hybrid_gpus, self.standalone_gpus = max(1, int(total_gpus)), int(hybrid_gpus), int(standalone_gpus)
        self.reset()

    def reset(self) -> None:
        self.values: dict[str, list[float]] = {}
        self.sample_counts: list[int] = []
        self.timestamps: list[float] = []

    @property
    def step_count(self) -> int:
        return len(self.sample_counts)

    def add_step_metrics(self, metrics: dict, sample_count: int = 1, timestamp: float = None) -> None:
        import time

        self.sample_counts.append(int(sample_count))
        self.timestamps.append(time.time() if timestamp is None else float(timestamp))
        for k, v in metrics.items():
            if hasattr(v, "item") and getattr(v, "numel", lambda: 1)() == 1:
                v = v.item()
            if isinstance(v, (int, float, np.floating, np.integer)) and not isinstance(v, bool):
                self.values.setdefault(k, []).append(float(v))

    @classmethod
    def rule(cls, name: str) -> str:
        if name in cls.LAST:
            return "last"
        if name in cls.SUM:
            return "sum"
        if name in cls.BY_SUFFIX:
            return cls.BY_SUFFIX[name]
        low = name.lower()
        if "timing_s/" in low:
            return "sum"
        if "weighted_avg" in low:
            return "weighted"
        for words, how in ((("mean", "avg", "average"), "mean"), (("max",), "max"), (("min",), "min"), (("sum", "total"), "sum")):
            if any(w in low for w in words):
                return how
        return "mean"

    def _reduce(self, name: str, vals: list[float]) -> float:
        how = self.rule(name)
        if how == "last":
            return vals[-1]
        if how == "sum":
            return float(sum(vals))
        if how == "max":
            return max(vals)
        if how == "min":
            return min(vals)
        if how == "weighted" and len(vals) == len(self.sample_counts) and sum(self.sample_counts) > 0:
            return sum(v * c for v, c in zip(vals, self.sample_counts)) / sum(self.sample_counts)
        return sum(vals) / len(vals)

    def get_aggregated_metrics(self, rollout_resource_utilization: float = None) -> dict[str, float]:
        if not self.sample_counts:
            return {}
        out = {k: self._reduce(k, v) for k, v in self.values.items() if v}
        if "global_seqlen/minmax_diff" in out and {"global_seqlen/max", "global_seqlen/min"} <= set(out):
            out["global_seqlen/minmax_diff"] = out["global_seqlen/max"] - out["global_seqlen/min"]
        if {"perf/throughput", "perf/total_num_tokens", "perf/time_per_step"} <= set(out) and out["perf/time_per_step"] > 0:
            out["perf/throughput"] = out["perf/total_num_tokens"] / (out["perf/time_per_step"] * self.total_gpus)
        if out.get("timing_s/step", 0.0) > 0 and "timing_s/gen" in out:
            out["fully_async/trainer/idle_ratio"] = out["timing_s/gen"] / out["timing_s/step"]
        alloc = out.get("dynamic_resource/train_allocated_time_s", 0.0)
        if alloc > 0 and "dynamic_resource/train_compute_time_s" in out:
            out["dynamic_resource/train_resource_utilization"] = out["dynamic_resource/train_compute_time_s"] / alloc
        gpus = self.hybrid_gpus + self.standalone_gpus
        if ("dynamic_resource/train_resource_utilization" in out and rollout_resource_utilization is not None and gpus > 0
                and out.get("timing_s/step", 0.0) > 0):
            out["dynamic_resource/rollout_resource_utilization"] = float(rollout_resource_utilization)
            x = min(1.0, max(0.0, out.get("timing_s/wait_for_enough_samples", 0.0) / out["timing_s/step"]))
            a, b = self.hybrid_gpus, self.standalone_gpus
            out["dynamic_resource/resource_utilization"] = ((1 - x) * a * out["dynamic_resource/train_resource_utilization"]
                                                            + (x * a + b) * float(rollout_resource_utilization)) / gpus
        return out

    def get_current_stats(self) -> dict[str, Any]:
        return {"step_count": self.step_count, "metric_count": len(self.values), "total_samples": sum(self.sample_counts),
                "metric_names": sorted(self.values)}


def task_exception_handler(task) -> None:
    """Done-callback for background tasks: a task that died with an exception says so instead of vanishing."""
    import logging

    if task.cancelled():
        return
    exc = task.exception()
    if exc is not None:
        logging.getLogger(__name__).error("background task %s failed: %r", task.get_name(), exc, exc_info=exc)


def safe_create_task(coro, name: str, task_set: set = None):
    """``asyncio.create_task`` with a name, the exception reporter above, and membership in ``task_set`` while it runs (a
    task nobody holds a reference to may be collected before it finishes)."""
    import asyncio

    task = asyncio.get_event_loop().create_task(coro, name=name)
    task.add_done_callback(task_exception_handler)
    if task_set is not None:
        task_set.add(task)
        task.add_done_callback(task_set.discard)
    return task
