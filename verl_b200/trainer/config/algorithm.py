"""Algorithm-level configuration. Parity target: ``verl/trainer/config/algorithm.py`` (``KLControlConfig`` :24,
``FilterGroupsConfig`` :43, ``RolloutCorrectionConfig`` + presets :63-616, ``AlgoConfig`` :620-672)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ...base_config import BaseConfig

__all__ = ["KLControlConfig", "FilterGroupsConfig", "RolloutCorrectionConfig", "AlgoConfig"]


@dataclass
class KLControlConfig(BaseConfig):
    type: str = "fixed"
    kl_coef: float = 0.001
    horizon: int = 10000
    target_kl: float = 0.1


@dataclass
class FilterGroupsConfig(BaseConfig):
    enable: bool = False
    metric: Optional[str] = None
    max_num_gen_batches: int = 0


@dataclass
class RolloutCorrectionConfig(BaseConfig):
    """Importance-sampling (IS) and rejection-sampling (RS) correction between the rollout policy and the training
    policy. ``rollout_is``/``rollout_rs`` choose the aggregation level; ``bypass_mode`` reuses the rollout log-probs
    as the old log-probs (no extra forward pass); ``loss_type`` selects PPO-clip or REINFORCE in bypass mode."""

    rollout_is: Optional[str] = "sequence"  # token | sequence | null
    rollout_is_threshold: float = 2.0
    rollout_is_batch_normalize: bool = False
    rollout_rs: Optional[str] = None  # token_k1 | seq_sum_k1 | seq_mean_k1 | seq_max_k2 | geometric ...
    rollout_rs_threshold: Any = None
    bypass_mode: bool = False
    loss_type: str = "ppo_clip"

    # -- named presets -----------------------------------------------------------------------
    @classmethod
    def decoupled_token_is(cls, threshold: float = 2.0):
        return cls(rollout_is="token", rollout_is_threshold=threshold)

    @classmethod
    def decoupled_seq_is(cls, threshold: float = 2.0):
        return cls(rollout_is="sequence", rollout_is_threshold=threshold)

    @classmethod
    def decoupled_seq_is_rs(cls, is_threshold: float = 2.0, rs_threshold="0.5_2.0"):
        return cls(rollout_is="sequence", rollout_is_threshold=is_threshold, rollout_rs="seq_sum_k1", rollout_rs_threshold=rs_threshold)

    @classmethod
    def decoupled_geo_rs(cls, rs_threshold="0.999_1.001"):
        return cls(rollout_is=None, rollout_rs="seq_mean_k1", rollout_rs_threshold=rs_threshold)

    @classmethod
    def decoupled_geo_rs_token_tis(cls, is_threshold: float = 2.0, rs_threshold="0.999_1.001"):
        return cls(rollout_is="token", rollout_is_threshold=is_threshold, rollout_rs="seq_mean_k1", rollout_rs_threshold=rs_threshold)

    @classmethod
    def decoupled_k3_rs(cls, rs_threshold: float = 0.01):
        return cls(rollout_is=None, rollout_rs="seq_mean_k3", rollout_rs_threshold=rs_threshold)

    @classmethod
    def decoupled_k3_rs_token_tis(cls, is_threshold: float = 2.0, rs_threshold: float = 0.01):
        return cls(rollout_is="token", rollout_is_threshold=is_threshold, rollout_rs="seq_mean_k3", rollout_rs_threshold=rs_threshold)

    @classmethod
    def decoupled_token_rs(cls, rs_threshold="0.5_2.0"):
        return cls(rollout_is=None, rollout_rs="token_k1", rollout_rs_threshold=rs_threshold)

    @classmethod
    def bypass_ppo_clip(cls):
        return cls(rollout_is=None, rollout_rs=None, bypass_mode=True, loss_type="ppo_clip")

    @classmethod
    def bypass_ppo_clip_geo_rs(cls, rs_threshold="0.999_1.001"):
        return cls(rollout_is=None, rollout_rs="seq_mean_k1", rollout_rs_threshold=rs_threshold, bypass_mode=True, loss_type="ppo_clip")

    @classmethod
    def bypass_ppo_clip_k3_rs(cls, rs_threshold: float = 0.01):
        return cls(rollout_is=None, rollout_rs="seq_mean_k3", rollout_rs_threshold=rs_threshold, bypass_mode=True, loss_type="ppo_clip")

    @classmethod
    def bypass_pg_is(cls, threshold: float = 2.0):
        return cls(rollout_is="sequence", rollout_is_threshold=threshold, bypass_mode=True, loss_type="reinforce")

    @classmethod
    def bypass_pg_token_is(cls, threshold: float = 2.0):
        return cls(rollout_is="token", rollout_is_threshold=threshold, bypass_mode=True, loss_type="reinforce")

    @classmethod
    def bypass_pg_rs(cls, rs_threshold="0.999_1.001"):
        return cls(rollout_is=None, rollout_rs="seq_mean_k1", rollout_rs_threshold=rs_threshold, bypass_mode=True, loss_type="reinforce")

    @classmethod
    def bypass_pg_geo_rs(cls, rs_threshold="0.999_1.001"):
        return cls.bypass_pg_rs(rs_threshold)

    @classmethod
    def bypass_pg_geo_rs_token_tis(cls, is_threshold: float = 2.0, rs_threshold="0.999_1.001"):
        return cls(rollout_is="token", rollout_is_threshold=is_threshold, rollout_rs="seq_mean_k1",
                   rollout_rs_threshold=rs_threshold, bypass_mode=True, loss_type="reinforce")

    @classmethod
    def bypass_pg_k3_rs(cls, rs_threshold: float = 0.01):
        return cls(rollout_is=None, rollout_rs="seq_mean_k3", rollout_rs_threshold=rs_threshold, bypass_mode=True, loss_type="reinforce")

    @classmethod
    def bypass_pg_k3_rs_token_tis(cls, is_threshold: float = 2.0, rs_threshold: float = 0.01):
        return cls(rollout_is="token", rollout_is_threshold=is_threshold, rollout_rs="seq_mean_k3",
                   rollout_rs_threshold=rs_threshold, bypass_mode=True, loss_type="reinforce")

    @classmethod
    def disabled(cls):
        return cls(rollout_is=None, rollout_rs=None)


@dataclass
class AlgoConfig(BaseConfig):
    gamma: float = 1.0
    lam: float = 1.0
    adv_estimator: str = "gae"
    norm_adv_by_std_in_grpo: bool = True
    use_kl_in_reward: bool = False
    kl_penalty: str = "kl"
    kl_ctrl: KLControlConfig = field(default_factory=KLControlConfig)
    use_pf_ppo: bool = False
    pf_ppo: dict = field(default_factory=dict)
    filter_groups: Optional[FilterGroupsConfig] = None
    rollout_correction: Optional[RolloutCorrectionConfig] = None
    gdpo_reward_keys: Optional[list] = None
    gdpo_reward_weights: Optional[list] = None
