"""Reward-side configuration dataclasses. Parity target: ``verl/workers/config/reward.py`` (``RewardManagerConfig`` :32,
``SandboxFusionConfig`` :67, ``RewardModelConfig`` :82, ``RewardConfig`` :94)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ...base_config import BaseConfig

__all__ = ["RewardManagerConfig", "SandboxFusionConfig", "RewardModelConfig", "RewardConfig"]


@dataclass
class RewardManagerConfig(BaseConfig):
    """``source="register"``: ``name`` is looked up among the registered reward managers; ``source="importlib"``: ``name`` is a
    class in the user module ``module`` (``{path, name}``)."""

    source: str = "register"
    name: str = "naive"
    module: Optional[dict] = None

    def __post_init__(self):
        if self.source == "register":
            from ...experimental.reward_loop.reward_manager.registry import REWARD_LOOP_MANAGERS
            from ..reward_manager.registry import REWARD_MANAGER_REGISTRY as REWARD_MANAGERS
            from .. import reward_manager as _rm  # noqa: F401  (registers the built-in managers)
            from ...experimental.reward_loop import reward_manager as _rlm  # noqa: F401

            if self.name not in REWARD_MANAGERS and self.name not in REWARD_LOOP_MANAGERS:
                raise ValueError(f"Reward manager is not registered: name={self.name!r}, "
                                 f"registered: {sorted(set(REWARD_MANAGERS) | set(REWARD_LOOP_MANAGERS))}")
        elif self.source == "importlib":
            if not self.module or not (self.module.get("path") if hasattr(self.module, "get") else getattr(self.module, "path", None)):
                raise ValueError("reward_manager.source=importlib needs reward_manager.module.path")
        else:
            raise ValueError(f"unknown reward manager source {self.source!r} (register | importlib)")


@dataclass
class SandboxFusionConfig(BaseConfig):
    url: Optional[str] = None
    max_concurrent: int = 64
    memory_limit_mb: int = 1024


@dataclass
class RewardModelConfig(BaseConfig):
    enable: bool = False
    enable_resource_pool: bool = False
    n_gpus_per_node: int = 8
    nnodes: int = 0
    model_path: Optional[str] = None
    rollout: Any = None   # a RolloutConfig: how the reward model is served


@dataclass
class RewardConfig(BaseConfig):
    num_workers: int = 8
    reward_manager: RewardManagerConfig = field(default_factory=RewardManagerConfig)
    reward_model: RewardModelConfig = field(default_factory=RewardModelConfig)
    sandbox_fusion: SandboxFusionConfig = field(default_factory=SandboxFusionConfig)
    custom_reward_function: dict = field(default_factory=dict)
