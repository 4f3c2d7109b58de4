"""Engine configurations. Parity target: ``verl/workers/config/engine.py:149-662``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ...base_config import BaseConfig
from .checkpoint import CheckpointConfig
from .model import HFModelConfig
from .optimizer import OptimizerConfig

__all__ = ["EngineConfig", "FSDPEngineConfig", "McoreEngineConfig", "VeOmniEngineConfig", "TorchtitanEngineConfig",
           "AutomodelEngineConfig", "TrainingWorkerConfig"]


@dataclass
class EngineConfig(BaseConfig):
    _mutable_fields = {"use_dynamic_bsz", "max_token_len_per_gpu", "micro_batch_size_per_gpu",
                       "infer_max_token_len_per_gpu", "infer_micro_batch_size_per_gpu", "use_fused_kernels",
                       "use_remove_padding", "forward_only", "param_offload", "optimizer_offload"}
    strategy: str = "fsdp"
    param_offload: bool = False
    optimizer_offload: bool = False
    # which Adam state optimizer_offload keeps in pinned host memory: "moments" (exp_avg and exp_avg_sq) or one of the two
    # by name; every offloaded tensor crosses the host link twice per optimizer step, so offload no more than the
    # activations need
    optimizer_offload_states: str = "moments"
    grad_offload: bool = False
    forward_only: bool = False
    dtype: str = "bfloat16"
    seed: int = 42
    full_determinism: bool = False
    use_dynamic_bsz: bool = False
    max_token_len_per_gpu: int = 16384
    micro_batch_size_per_gpu: Optional[int] = None
    infer_max_token_len_per_gpu: int = 16384
    infer_micro_batch_size_per_gpu: Optional[int] = None
    use_fused_kernels: bool = True
    use_remove_padding: bool = True
    use_torch_compile: bool = False
    entropy_from_logits_with_chunking: bool = False
    entropy_checkpointing: bool = False
    qat: dict = field(default_factory=dict)            # {enable, mode: w4a16, group_size: 16, ignore_patterns}
    router_replay: dict = field(default_factory=dict)  # {mode: disabled | R2 | R3}


@dataclass
class FSDPEngineConfig(EngineConfig):
    """Sharded data-parallel engine. ``zero_stage=2`` (default): gradients and optimizer state are sharded over the
    data-parallel group while every GPU keeps a full bf16 working copy of the weights, which removes all parameter gathers
    from the forward / backward path and lets the colocated rollout engine read the weights in place. That fits 180 GB for
    dense models up to roughly 20 B parameters (2 bytes of weights + 4 bytes of transient fp32 gradients per parameter).
    ``zero_stage=3`` (the reference's FULL_SHARD): the working weights are sharded as well, per unit (embedding, each layer,
    head); a unit is gathered into one of two arenas while the previous unit computes, its gradients are reduce-scattered as
    the backward pass leaves it, and the rollout engine gets a gathered replica at every weight hand-over. Larger models can
    also shard with the tensor x pipeline x expert parallel engine (``strategy=megatron``)."""

    wrap_policy: dict = field(default_factory=dict)
    offload_policy: bool = False
    reshard_after_forward: bool = True
    fsdp_size: int = -1
    forward_prefetch: bool = False
    model_dtype: str = "fp32"
    use_orig_params: bool = False
    mixed_precision: Optional[dict] = None
    ulysses_sequence_parallel_size: int = 1
    # context parallelism: blocks of this many data-parallel ranks split the tokens of the same micro-batches and exchange
    # keys / values around attention (no constraint on the number of KV heads; exclusive with Ulysses)
    context_parallel_size: int = 1
    context_parallel_mode: str = "zigzag"   # zigzag (rank i holds chunks i and 2 cp - 1 - i of the stream: balanced causal work) | contiguous
    # a group size per row instead of one for the run: every row is cut over the smallest power-of-two group of the block's
    # ranks that keeps its share under max_seqlen_per_dp_cp_rank tokens (context_parallel_size = the block, a power of two)
    dynamic_context_parallel: bool = False
    max_seqlen_per_dp_cp_rank: int = 4096
    zero_stage: int = 2
    enable_gradient_checkpointing: bool = True
    enable_activation_offload: bool = False
    fused_comm: bool = True  # peer-memory fused reduce-scatter + AdamW + all-gather when symmetric memory is available
    # limit of the device-side barriers around the fused optimizer step: ranks do not talk during gradient accumulation, so
    # it has to cover the skew a whole mini-batch can build up; when it runs out the step is skipped on every rank
    peer_barrier_timeout_s: float = 120.0
    # option tree of the ``fsdp_turbo`` strategy (``workers/engine/native/turbo.py`` lists the keys that have an effect)
    turbo_config: dict = field(default_factory=dict)
    strategy: str = "fsdp"

    def __post_init__(self):
        assert self.strategy in ("fsdp", "fsdp2", "fsdp_turbo"), f"strategy {self.strategy} not supported"
        if int(self.zero_stage) not in (2, 3):
            raise NotImplementedError("zero_stage must be 2 (replicated bf16 working weights, sharded gradients and optimizer "
                                      "state) or 3 (working weights sharded per layer as well)")


@dataclass
class McoreEngineConfig(EngineConfig):
    tensor_model_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    pipeline_schedule: str = "1f1b"   # 1f1b | gpipe (all forwards, then all backwards)
    vocab_parallel_head: bool = True    # LM head rows split over the tensor-parallel group
    expert_tensor_parallel_size: Optional[int] = None
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: Optional[int] = None
    context_parallel_size: int = 1
    context_parallel_mode: str = "zigzag"
    sequence_parallel: bool = True      # token-sliced residual stream inside the tensor-parallel group (on with TP > 1)
    use_distributed_optimizer: bool = True
    use_dist_checkpointing: bool = False
    dist_checkpointing_path: Optional[str] = None
    dynamic_context_parallel: bool = False
    override_transformer_config: dict = field(default_factory=dict)
    override_ddp_config: dict = field(default_factory=dict)
    use_mbridge: bool = False
    enable_gradient_checkpointing: bool = True
    strategy: str = "megatron"

    def __post_init__(self):
        if self.tensor_model_parallel_size == 1:
            object.__setattr__(self, "sequence_parallel", False)


@dataclass
class VeOmniEngineConfig(FSDPEngineConfig):
    """Option names of the reference's VeOmni backend (``verl/workers/config/engine.py:308-443``); translated onto the
    engines of this framework by ``workers/engine/backends.py``."""

    ulysses_parallel_size: int = 1
    expert_parallel_size: int = 1
    enable_full_shard: bool = False
    enable_fsdp_offload: bool = False
    enable_reentrant: bool = False
    init_device: str = "meta"
    attn_implementation: str = "flash_attention_2"
    moe_implementation: str = "fused"
    activation_gpu_limit: float = 0.0
    strategy: str = "veomni"

    def __post_init__(self):
        pass


@dataclass
class TorchtitanEngineConfig(EngineConfig):
    """Option names of the reference's TorchTitan backend (``verl/workers/config/engine.py:461-523``)."""

    wrap_policy: dict = field(default_factory=dict)
    reshard_after_forward: str = "default"   # default | always | never
    offload_policy: bool = False
    data_parallel_size: int = 1
    data_parallel_shard_size: int = -1
    data_parallel_replicate_size: int = 1
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1
    expert_tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    context_parallel_size: int = 1
    attn_type: str = "flex"
    activation_checkpoint: str = "selective"   # none | selective | full
    max_seq_len: Optional[int] = None
    strategy: str = "torchtitan"


@dataclass
class AutomodelEngineConfig(EngineConfig):
    """Option names of the reference's NeMo-Automodel backend (``verl/workers/config/engine.py:540-650``); the long names
    are kept as synonyms of ``tp_size`` / ``cp_size`` / ``ep_size``."""

    distributed_strategy: str = "fsdp2"
    tp_size: int = 1
    pp_size: int = 1
    cp_size: int = 1
    ep_size: int = 1
    dp_replicate_size: int = 1
    sequence_parallel: bool = False
    activation_checkpointing: bool = False
    tensor_parallel_size: int = 1
    context_parallel_size: int = 1
    expert_parallel_size: int = 1
    model_dtype: str = "fp32"
    attn_implementation: str = "flash_attention_2"
    backend_config: dict = field(default_factory=dict)
    moe_config: dict = field(default_factory=dict)
    strategy: str = "automodel"


@dataclass
class TrainingWorkerConfig(BaseConfig):
    model_type: str = "language_model"  # language_model | value_model
    model_config: Any = None
    engine_config: Any = None
    optimizer_config: Any = None
    checkpoint_config: Any = None
    profiler_config: Any = None
    auto_select_engine_optim_fn: Any = None
