"""Optimizer configuration. Parity target: ``verl/workers/config/optimizer.py:298-351``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ...base_config import BaseConfig

__all__ = ["OptimizerConfig", "FSDPOptimizerConfig", "McoreOptimizerConfig", "build_optimizer", "lr_at_step"]


@dataclass
class OptimizerConfig(BaseConfig):
    _mutable_fields = {"clip_grad", "total_training_steps", "lr_warmup_steps"}
    lr: float = 1e-6
    lr_warmup_steps_ratio: float = 0.0
    lr_warmup_steps: Optional[int] = -1
    total_training_steps: int = -1
    weight_decay: float = 0.01
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    clip_grad: float = 1.0
    optimizer: str = "AdamW"
    optimizer_impl: str = "verl_b200.fused"
    lr_scheduler_type: str = "constant"  # constant | cosine | wsd
    min_lr_ratio: float = 0.0
    num_cycles: float = 0.5
    override_optimizer_config: Optional[dict] = None
    # Muon (``optimizer: muon``): momentum + Newton-Schulz orthogonalisation for the 2-D weights of the layers, AdamW
    # (with the fields above) for embeddings, heads, norms and biases
    muon_momentum: float = 0.95
    muon_nesterov: bool = False
    muon_split_qkv: bool = True
    muon_scale_mode: str = "spectral"          # spectral | shape_scaling | unit_rms_norm | none
    muon_coefficient_type: str = "quintic"     # quintic | simple
    muon_num_ns_steps: int = 5
    muon_tp_mode: str = "blockwise"            # tensor-parallel shards are orthogonalised one by one
    muon_extra_scale_factor: float = 1.0
    muon_scalar_optimizer: str = "adam"
    muon_match_adamw_update_rms: bool = False  # extra factor = sqrt((1 - beta1) / (1 + beta1)): reuse an AdamW learning rate

    def __post_init__(self):
        assert self.lr != "???", "optimizer lr must be set"
        assert self.lr_scheduler_type in ("constant", "cosine", "wsd")
        if self.muon_match_adamw_update_rms:
            assert self.muon_extra_scale_factor == 1.0, "muon_match_adamw_update_rms derives muon_extra_scale_factor: set only one"
        assert self.muon_tp_mode == "blockwise" and str(self.muon_scalar_optimizer).lower() in ("adam", "adamw")

    @property
    def muon_update_scale(self) -> float:
        """Factor on the learning rate of the orthogonalised updates."""
        if self.muon_match_adamw_update_rms:
            from ..engine.native.muon import adamw_rms_match_scale_factor

            return adamw_rms_match_scale_factor(float(self.betas[0]))
        return float(self.muon_extra_scale_factor)


@dataclass
class FSDPOptimizerConfig(OptimizerConfig):
    warmup_style: Optional[str] = None  # deprecated alias of lr_scheduler_type

    def __post_init__(self):
        if self.warmup_style is not None:
            object.__setattr__(self, "lr_scheduler_type", self.warmup_style)
        super().__post_init__()


@dataclass
class McoreOptimizerConfig(OptimizerConfig):
    lr_warmup_init: float = 0.0
    lr_decay_steps: Optional[int] = None
    lr_decay_style: str = "constant"
    min_lr: float = 0.0
    use_distributed_optimizer: bool = True


def lr_at_step(cfg: OptimizerConfig, step: int) -> float:
    """Learning rate for optimizer step ``step`` (0-based)."""
    from ...utils.torch_functional import cosine_factor, wsd_factor

    total = cfg.total_training_steps if cfg.total_training_steps and cfg.total_training_steps > 0 else 1
    warm = cfg.lr_warmup_steps if (cfg.lr_warmup_steps is not None and cfg.lr_warmup_steps >= 0) else int(
        cfg.lr_warmup_steps_ratio * total)
    if cfg.lr_scheduler_type == "cosine":
        return cfg.lr * cosine_factor(step, warm, total, cfg.min_lr_ratio, cfg.num_cycles)
    if cfg.lr_scheduler_type == "wsd":
        return cfg.lr * wsd_factor(step, warm, total, min_ratio=cfg.min_lr_ratio)
    return cfg.lr * (min(1.0, step / max(1, warm)) if warm > 0 else 1.0)


def build_optimizer(parameters, config: OptimizerConfig):
    """torch optimizer for plain ``nn.Parameter`` lists (used by the CPU reference path and LoRA adapters)."""
    import torch

    cls = getattr(torch.optim, config.optimizer)
    kw = dict(lr=config.lr, weight_decay=config.weight_decay)
    if "Adam" in config.optimizer:
        kw.update(betas=tuple(config.betas), eps=config.eps)
    kw.update(config.override_optimizer_config or {})
    return cls(parameters, **kw)
