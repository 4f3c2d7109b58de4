"""Decision rules of the hybrid mode of a split job (trainer GPUs that generate while the trainer would wait).

``AdaptiveSwitchThreshold``: how many prompt groups must be ready before the lent GPUs return to training. It starts at
``switch_threshold_ratio`` x the training batch, never below one mini-batch nor above the batch, and adapts: steps in which
the trainer still had to wait push it up (go back later, generate more), steps without waiting pull it down, each only after
``switch_threshold_release_steps`` such steps in a row.

``SwitchCostWindow`` / ``switch_is_worth_it``: lending pays when the waiting it saves exceeds what the two mode changes
cost: ``remaining samples x seconds per sample x (1 - 1 / scaling factor) > cost to rollout + cost to trainer`` (mean of the
last few switches each; unknown cost or unknown rate: switch, to learn them).

Parity target: ``verl/trainer/ppo/v1/trainer_separate_async.py:261-330``.
"""

from __future__ import annotations

from collections import deque
from typing import Optional

from ...config.config import HybridRolloutSwitchConfig

__all__ = ["AdaptiveSwitchThreshold", "SwitchCostWindow", "switch_is_worth_it"]


class AdaptiveSwitchThreshold:
    def __init__(self, config: HybridRolloutSwitchConfig, train_batch_size: int, parameter_sync_step: int = 1):
        self.cfg = config
        self.batch, self.rounds = int(train_batch_size), max(1, int(parameter_sync_step))
        self.ratio = float(config.switch_threshold_ratio)
        self._idle = self._calm = 0

    def threshold(self) -> int:
        mini = self.batch // self.rounds
        return min(max(round(self.ratio * self.batch), mini), self.batch)

    def adapt(self, had_idle: bool) -> float:
        c = self.cfg
        if not c.adaptive_switch_threshold:
            return self.ratio
        if had_idle:
            self._calm = 0
            self._idle = min(self._idle + 1, c.switch_threshold_release_steps)
            if self._idle >= c.switch_threshold_release_steps:
                self.ratio = min(1.0, self.ratio + c.switch_threshold_step_up)
        else:
            self._idle = 0
            self._calm = min(self._calm + 1, c.switch_threshold_release_steps)
            if self._calm >= c.switch_threshold_release_steps:
                self.ratio = max(1.0 / self.rounds, self.ratio - c.switch_threshold_step_down)
        return self.ratio


class SwitchCostWindow:
    def __init__(self, size: int = 3):
        self.to_rollout: deque = deque(maxlen=int(size))
        self.to_trainer: deque = deque(maxlen=int(size))

    def effective_cost(self) -> Optional[float]:
        if not self.to_rollout or not self.to_trainer:
            return None
        return sum(self.to_rollout) / len(self.to_rollout) + sum(self.to_trainer) / len(self.to_trainer)


def switch_is_worth_it(remaining: int, seconds_per_sample: Optional[float], scaling_factor: float, cost_s: Optional[float]) -> bool:
    """``scaling_factor``: generation capacity with the lent GPUs over capacity without them (> 1)."""
    if remaining <= 0:
        return False
    if seconds_per_sample is None or cost_s is None:
        return True
    return remaining * seconds_per_sample * (1.0 - 1.0 / max(scaling_factor, 1.0 + 1e-9)) > cost_s
