"""Small configuration dataclasses of the trainer. Parity target: ``verl/trainer/config/config.py`` (``CheckpointConfig``
:24, ``ProfileConfig`` :55, ``HybridRolloutSwitchConfig`` :74, ``BaseModelConfig`` :93, ``ModuleConfig`` :115)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ...base_config import BaseConfig
from ...workers.config.checkpoint import CheckpointConfig

__all__ = ["CheckpointConfig", "ProfileConfig", "HybridRolloutSwitchConfig", "BaseModelConfig", "ModuleConfig"]


@dataclass
class ProfileConfig(BaseConfig):
    profile_ranks: Optional[list] = None   # None: every rank
    step_start: int = -1
    step_end: int = -1
    save_path: Optional[str] = None


@dataclass
class HybridRolloutSwitchConfig(BaseConfig):
    """When trainer GPUs of a split job lend themselves to generation. ``switch_threshold_ratio``: the share of a training
    batch that must be ready in the replay buffer before the GPUs go back to training; with ``adaptive_switch_threshold`` it
    moves up by ``switch_threshold_step_up`` after ``switch_threshold_release_steps`` consecutive steps in which the trainer
    had to wait for samples, and down by ``switch_threshold_step_down`` after as many steps without waiting.
    ``switch_cost_window_size``: how many recent switches the cost estimate averages over."""

    enable_switch: bool = False
    switch_threshold_ratio: float = 0.4
    adaptive_switch_threshold: bool = True
    switch_threshold_step_up: float = 0.05
    switch_threshold_step_down: float = 0.03
    switch_threshold_release_steps: int = 2
    switch_cost_window_size: int = 3

    def __post_init__(self):
        if not 0.0 < self.switch_threshold_ratio <= 1.0:
            raise ValueError(f"switch_threshold_ratio must be in (0, 1], got {self.switch_threshold_ratio}")
        if self.switch_cost_window_size <= 0:
            raise ValueError("switch_cost_window_size must be positive")


@dataclass
class BaseModelConfig(BaseConfig):
    path: str = "~/models/deepseek-llm-7b-chat"
    tokenizer_path: Optional[str] = None
    override_config: dict = field(default_factory=dict)
    external_lib: Optional[str] = None
    trust_remote_code: bool = False
    lora: dict = field(default_factory=dict)


@dataclass
class ModuleConfig(BaseConfig):
    """A user module: ``path`` of a file to execute and / or ``name`` to import it under."""

    path: Optional[str] = None
    name: Optional[str] = None
