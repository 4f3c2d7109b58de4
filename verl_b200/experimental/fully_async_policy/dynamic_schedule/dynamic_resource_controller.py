"""How many of the elastic replicas serve rollout right now.

A job has ``fixed_rollout`` replicas that always generate and ``elastic`` replicas (GPUs of the trainer pool that can
be lent). After every trainer step the controller receives what was measured (queue depth, trainer idle seconds,
trainer step seconds, rollout throughput) and a policy answers with the target number of lent replicas; the
controller turns the difference into ``add_replicas`` / ``remove_replicas`` calls on the rollouter.

Parity target: ``verl/experimental/fully_async_policy/dynamic_schedule/dynamic_resource_controller.py:51`` and the
policies ``DefaultDynamicSchedulePolicy`` / ``FixedRatioDynamicSchedulePolicy`` / ``StaticFullyAsyncPolicy``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

__all__ = ["ScheduleObservation", "StaticFullyAsyncPolicy", "FixedRatioDynamicSchedulePolicy",
           "DefaultDynamicSchedulePolicy", "DynamicResourceController"]


@dataclass
class ScheduleObservation:
    queue_size: int            # finished samples waiting for the trainer
    required_samples: int      # samples the trainer needs per step
    trainer_idle_s: float      # time the last step spent waiting for samples
    trainer_step_s: float      # time the last step spent training
    lent: int                  # elastic replicas currently serving rollout
    elastic: int               # elastic replicas in total


class StaticFullyAsyncPolicy:
    """Never lends anything: the split chosen at launch stays."""

    def target(self, obs: ScheduleObservation) -> int:
        return 0


class FixedRatioDynamicSchedulePolicy:
    """Lends a fixed share of the elastic replicas whenever the trainer had to wait at all."""

    def __init__(self, ratio: float = 0.5):
        self.ratio = ratio

    def target(self, obs: ScheduleObservation) -> int:
        return int(round(self.ratio * obs.elastic)) if obs.trainer_idle_s > 0 else 0


class DefaultDynamicSchedulePolicy:
    """Hysteresis controller on the trainer's idle fraction: lend one more replica when the trainer idles more than
    ``high`` of its step and the queue cannot cover the next step; take one back when idling drops under ``low`` or
    the queue holds more than ``backlog_steps`` steps of samples."""

    def __init__(self, high: float = 0.2, low: float = 0.05, backlog_steps: float = 2.0):
        self.high, self.low, self.backlog_steps = high, low, backlog_steps

    def target(self, obs: ScheduleObservation) -> int:
        total = obs.trainer_idle_s + obs.trainer_step_s
        idle_frac = obs.trainer_idle_s / total if total > 0 else 0.0
        if obs.queue_size > self.backlog_steps * obs.required_samples or idle_frac < self.low:
            return max(0, obs.lent - 1)
        if idle_frac > self.high and obs.queue_size < obs.required_samples:
            return min(obs.elastic, obs.lent + 1)
        return obs.lent


class DynamicResourceController:
    def __init__(self, policy, elastic: int, add_fn: Optional[Callable[[int], None]] = None,
                 remove_fn: Optional[Callable[[int], None]] = None):
        self.policy, self.elastic = policy, int(elastic)
        self.add_fn, self.remove_fn = add_fn, remove_fn
        self.lent = 0
        self.history: list[int] = []

    def step(self, queue_size: int, required_samples: int, trainer_idle_s: float, trainer_step_s: float) -> int:
        obs = ScheduleObservation(queue_size, required_samples, trainer_idle_s, trainer_step_s, self.lent, self.elastic)
        tgt = max(0, min(self.elastic, int(self.policy.target(obs))))
        if tgt > self.lent and self.add_fn is not None:
            self.add_fn(tgt - self.lent)
        elif tgt < self.lent and self.remove_fn is not None:
            self.remove_fn(self.lent - tgt)
        self.lent = tgt
        self.history.append(tgt)
        return tgt
