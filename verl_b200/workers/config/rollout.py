"""Rollout configuration. Parity target: ``verl/workers/config/rollout.py`` (342 lines) and ``rollout.yaml``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ...base_config import BaseConfig

__all__ = ["SamplingConfig", "MultiTurnConfig", "AgentLoopConfig", "CheckpointEngineConfig", "RolloutConfig",
           "ServerConfig", "TraceConfig"]


@dataclass
class SamplingConfig(BaseConfig):
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    do_sample: bool = True
    n: int = 1


@dataclass
class MultiTurnConfig(BaseConfig):
    _mutable_fields = {"max_assistant_turns", "max_user_turns"}
    enable: bool = False
    max_assistant_turns: Optional[int] = None
    tool_config_path: Optional[str] = None
    function_tool_path: Optional[str] = None   # a Python file whose @function_tool functions become tools
    max_user_turns: Optional[int] = None
    max_parallel_calls: int = 1
    max_tool_response_length: int = 256
    tool_response_truncate_side: str = "middle"
    interaction_config_path: Optional[str] = None
    use_inference_chat_template: bool = False
    tokenization_sanity_check_mode: str = "strict"
    format: str = "hermes"
    num_repeat_rollouts: Optional[int] = None


@dataclass
class TraceConfig(BaseConfig):
    backend: Optional[str] = None
    token2text: bool = False
    max_samples_per_step_per_worker: Optional[int] = None


@dataclass
class AgentLoopConfig(BaseConfig):
    num_workers: int = 8
    default_agent_loop: str = "single_turn_agent"
    agent_loop_config_path: Optional[str] = None
    custom_async_server: dict = field(default_factory=dict)


@dataclass
class CheckpointEngineConfig(BaseConfig):
    backend: str = "naive"
    update_weights_bucket_megabytes: int = 2048
    engine_kwargs: dict = field(default_factory=dict)


@dataclass
class ServerConfig(BaseConfig):
    timeout: float = 60.0
    max_attempts: int = 3
    retry_delay: float = 2.0
    max_connections: int = 1000
    max_start_wait_time: float = 300.0


@dataclass
class RolloutConfig(BaseConfig):
    _mutable_fields = {"max_model_len", "load_format", "n"}
    name: str = "native"
    mode: str = "async"
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    do_sample: bool = True
    n: int = 1
    repetition_penalty: float = 1.0
    over_sample_rate: float = 0.0
    prompt_length: int = 512
    response_length: int = 512
    dtype: str = "bfloat16"
    gpu_memory_utilization: float = 0.5
    ignore_eos: bool = False
    enforce_eager: bool = False
    cudagraph_capture_sizes: Optional[list] = None
    free_cache_engine: bool = True
    data_parallel_size: int = 1
    expert_parallel_size: int = 1
    tensor_model_parallel_size: int = 2
    pipeline_model_parallel_size: int = 1
    max_num_batched_tokens: int = 8192
    max_model_len: Optional[int] = None
    max_num_seqs: int = 256
    logprobs_mode: str = "processed_logprobs"
    scheduling_policy: str = "fcfs"
    load_format: str = "dummy"
    log_prob_micro_batch_size: Optional[int] = None
    log_prob_micro_batch_size_per_gpu: Optional[int] = None
    log_prob_use_dynamic_bsz: bool = False
    log_prob_max_token_len_per_gpu: int = 16384
    disable_log_stats: bool = True
    multi_stage_wake_up: bool = False
    engine_kwargs: dict = field(default_factory=dict)
    calculate_log_probs: bool = False
    agent: AgentLoopConfig = field(default_factory=AgentLoopConfig)
    trace: TraceConfig = field(default_factory=TraceConfig)
    multi_turn: MultiTurnConfig = field(default_factory=MultiTurnConfig)
    server: ServerConfig = field(default_factory=ServerConfig)
    checkpoint_engine: CheckpointEngineConfig = field(default_factory=CheckpointEngineConfig)
    val_kwargs: SamplingConfig = field(default_factory=lambda: SamplingConfig(temperature=0.0, do_sample=False))
    update_weights_bucket_megabytes: int = 512
    skip_rollout: bool = False
    skip_dump_dir: str = "/tmp/rollout_dump"
    skip_tokenizer_init: bool = True
    enable_chunked_prefill: bool = True
    enable_prefix_caching: bool = False
    # inference servers that already run elsewhere (name: sglang | openai | trtllm | http): one replica per address
    server_urls: list = field(default_factory=list)
    server_dialect: Optional[str] = None
    served_model_name: Optional[str] = None
    server_timeout: float = 600.0
    server_api_key: Optional[str] = None
    prometheus: dict = field(default_factory=dict)
    quantization: Optional[str] = None  # None | fp8
    quantization_config_file: Optional[str] = None
    enable_rollout_routing_replay: bool = False
    enable_sleep_mode: bool = True
    layered_summon: bool = False
    block_size: int = 64
    sync_interval: int = 16
    profiler: dict = field(default_factory=dict)
    mtp: dict = field(default_factory=dict)
    disaggregation: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.expert_parallel_size > 1:
            assert self.expert_parallel_size == self.tensor_model_parallel_size * self.data_parallel_size, \
                "expert_parallel_size must equal tensor_model_parallel_size * data_parallel_size"
        if self.pipeline_model_parallel_size > 1 and self.name in ("native",):
            raise NotImplementedError("pipeline parallel rollout is not supported by the native engine")
