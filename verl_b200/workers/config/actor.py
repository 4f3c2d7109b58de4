"""Actor / reference / critic worker configuration.

Parity target: ``verl/workers/config/actor.py:105-343`` and ``critic.py``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ...base_config import BaseConfig
from .checkpoint import CheckpointConfig
from .engine import FSDPEngineConfig, McoreEngineConfig
from .optimizer import OptimizerConfig

__all__ = ["PolicyLossConfig", "ActorConfig", "FSDPActorConfig", "McoreActorConfig", "RefConfig", "CriticConfig",
           "FSDPCriticConfig", "McoreCriticConfig"]


@dataclass
class PolicyLossConfig(BaseConfig):
    loss_mode: str = "vanilla"
    clip_cov_ratio: float = 0.0002
    clip_cov_lb: float = 1.0
    clip_cov_ub: float = 5.0
    kl_cov_ratio: float = 0.0002
    ppo_kl_coef: float = 0.1
    dro_beta: Optional[float] = None
    rollout_correction: Optional[dict] = None


@dataclass
class ActorConfig(BaseConfig):
    _mutable_fields = {"ppo_mini_batch_size", "ppo_micro_batch_size", "ppo_micro_batch_size_per_gpu",
                       "ppo_infer_micro_batch_size_per_gpu", "engine", "model_config", "global_batch_info",
                       "calculate_sum_pi_squared"}
    strategy: str = "fsdp"
    ppo_mini_batch_size: int = 256
    ppo_micro_batch_size: Optional[int] = None
    ppo_micro_batch_size_per_gpu: Optional[int] = None
    ppo_infer_micro_batch_size_per_gpu: Optional[int] = None
    use_dynamic_bsz: bool = False
    ppo_max_token_len_per_gpu: int = 16384
    ppo_infer_max_token_len_per_gpu: int = 16384
    clip_ratio: float = 0.2
    clip_ratio_low: float = 0.2
    clip_ratio_high: float = 0.2
    clip_ratio_c: float = 3.0
    tau_pos: float = 1.0
    tau_neg: float = 1.05
    freeze_vision_tower: bool = False
    policy_loss: PolicyLossConfig = field(default_factory=PolicyLossConfig)
    loss_agg_mode: str = "token-mean"
    loss_scale_factor: Optional[int] = None
    entropy_coeff: float = 0.0
    calculate_entropy: bool = False
    use_kl_loss: bool = False
    kl_loss_coef: float = 0.001
    kl_loss_type: str = "low_var_kl"
    ppo_epochs: int = 1
    shuffle: bool = False
    data_loader_seed: int = 1
    use_torch_compile: bool = False
    use_fused_kernels: bool = True
    use_remove_padding: bool = True
    calculate_sum_pi_squared: bool = False
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    optim: OptimizerConfig = field(default_factory=OptimizerConfig)
    engine: Any = None
    model_config: Any = None
    global_batch_info: dict = field(default_factory=dict)
    rollout_n: int = 1
    profiler: dict = field(default_factory=dict)
    router_replay: dict = field(default_factory=dict)

    def __post_init__(self):
        assert self.strategy != "???"
        assert self.loss_agg_mode in ("token-mean", "token-sum", "seq-mean-token-sum", "seq-mean-token-mean",
                                      "seq-mean-token-sum-norm"), f"Invalid loss_agg_mode: {self.loss_agg_mode}"
        if not self.use_dynamic_bsz and self.ppo_micro_batch_size is not None and self.ppo_micro_batch_size_per_gpu is not None:
            raise ValueError("[actor] set only one of ppo_micro_batch_size / ppo_micro_batch_size_per_gpu")

    def validate(self, n_gpus: int, train_batch_size: int, model_config=None) -> None:
        if not self.use_dynamic_bsz:
            if train_batch_size < self.ppo_mini_batch_size:
                raise ValueError(f"train_batch_size ({train_batch_size}) must be >= ppo_mini_batch_size "
                                 f"({self.ppo_mini_batch_size})")
            if self.ppo_micro_batch_size_per_gpu is not None:
                per = self.ppo_mini_batch_size * self.rollout_n // max(1, n_gpus)
                if per % self.ppo_micro_batch_size_per_gpu != 0 and per > self.ppo_micro_batch_size_per_gpu:
                    raise ValueError(f"per-GPU mini batch ({per}) must be divisible by ppo_micro_batch_size_per_gpu "
                                     f"({self.ppo_micro_batch_size_per_gpu})")


@dataclass
class FSDPActorConfig(ActorConfig):
    strategy: str = "fsdp"
    grad_clip: float = 1.0
    ulysses_sequence_parallel_size: int = 1
    entropy_from_logits_with_chunking: bool = False
    entropy_checkpointing: bool = False
    fsdp_config: FSDPEngineConfig = field(default_factory=FSDPEngineConfig)
    use_remove_padding: bool = True

    def __post_init__(self):
        super().__post_init__()
        if self.engine is None:
            object.__setattr__(self, "engine", self.fsdp_config)


@dataclass
class McoreActorConfig(ActorConfig):
    strategy: str = "megatron"
    megatron: McoreEngineConfig = field(default_factory=McoreEngineConfig)
    load_weight: bool = True

    def __post_init__(self):
        super().__post_init__()
        if self.engine is None:
            object.__setattr__(self, "engine", self.megatron)


@dataclass
class RefConfig(BaseConfig):
    strategy: str = "fsdp"
    log_prob_micro_batch_size: Optional[int] = None
    log_prob_micro_batch_size_per_gpu: Optional[int] = None
    log_prob_use_dynamic_bsz: bool = False
    log_prob_max_token_len_per_gpu: int = 16384
    fsdp_config: FSDPEngineConfig = field(default_factory=lambda: FSDPEngineConfig(forward_only=True))
    megatron: McoreEngineConfig = field(default_factory=lambda: McoreEngineConfig(forward_only=True))
    use_torch_compile: bool = False
    ulysses_sequence_parallel_size: int = 1
    profiler: dict = field(default_factory=dict)


@dataclass
class CriticConfig(BaseConfig):
    _mutable_fields = {"ppo_micro_batch_size_per_gpu", "ppo_mini_batch_size", "ppo_micro_batch_size", "model_config",
                       "engine", "global_batch_info"}
    strategy: str = "fsdp"
    enable: Optional[bool] = None
    ppo_micro_batch_size_per_gpu: Optional[int] = None
    ppo_micro_batch_size: Optional[int] = None
    ppo_mini_batch_size: int = 256
    use_dynamic_bsz: bool = False
    ppo_max_token_len_per_gpu: int = 32768
    forward_max_token_len_per_gpu: int = 32768
    forward_micro_batch_size_per_gpu: Optional[int] = None
    ppo_epochs: int = 1
    shuffle: bool = False
    data_loader_seed: int = 1
    cliprange_value: float = 0.5
    loss_agg_mode: str = "token-mean"
    rollout_n: int = 1
    optim: OptimizerConfig = field(default_factory=lambda: OptimizerConfig(lr=1e-5))
    model: Any = None
    model_config: Any = None
    engine: Any = None
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    global_batch_info: dict = field(default_factory=dict)
    profiler: dict = field(default_factory=dict)


@dataclass
class FSDPCriticConfig(CriticConfig):
    strategy: str = "fsdp"
    grad_clip: float = 1.0
    ulysses_sequence_parallel_size: int = 1
    fsdp_config: FSDPEngineConfig = field(default_factory=FSDPEngineConfig)


@dataclass
class McoreCriticConfig(CriticConfig):
    strategy: str = "megatron"
    megatron: McoreEngineConfig = field(default_factory=McoreEngineConfig)
