"""``fsdp_turbo`` backend: the sharded data-parallel engine in its fully sharded, fused configuration.

The reference's class of this name swaps PyTorch FSDP for an external fused FSDP runtime and reads that runtime's own
option tree (``turbo_config``). Here the same name selects what this framework has in that place: working weights sharded
per unit (``zero_stage=3``) and gathered by the GEMM kernels' own copy warps over peer memory while the previous unit
computes, gradients reduce-scattered as the backward pass leaves a unit, the optimizer step fused with the publication of
the new bf16 shard. The option tree is honoured where it has a meaning for this engine:

=============================================  ==========================================================================
``turbo_config`` key                           effect
=============================================  ==========================================================================
``distributed.fully_shard_parallel_size``      ``fsdp_size`` (hybrid sharding when smaller than the data-parallel size)
``distributed.ulysses_parallel_size``          ``ulysses_sequence_parallel_size`` (setting both is an error, as upstream)
``distributed.fsdp_plan.cpu_offload``          optimizer state in pinned host memory; taken from ``offload_policy``
``distributed.fsdp_plan.reshard_after_forward``  ``reshard_after_forward``
``distributed.fsdp_plan.param_dtype``          must be ``bf16`` (the working copy); ``reduce_dtype`` must be ``fp32``
``distributed.tensor_parallel_size`` / ``expert_parallel_size`` > 1   refused: those layouts are ``strategy=megatron`` here
=============================================  ==========================================================================

Keys that only tune the external runtime's prefetcher (``num_to_forward_prefetch`` ...) are accepted and have no effect: one
unit is always in flight.

Parity target: ``verl/workers/engine/fsdp/fsdp_turbo_impl.py`` (class :26, ``_init_parallel_state`` :31-42,
``_process_ulysses_config`` :72-83) and ``verl/trainer/config/engine/fsdp.yaml`` (``turbo_config`` :108-).
"""

from __future__ import annotations

import copy
from typing import Any, Optional

import torch.distributed as dist

from ..base import EngineRegistry
from .engine import NativeEngineWithLMHead, NativeEngineWithValueHead

__all__ = ["resolve_turbo_config", "NativeTurboEngineWithLMHead", "NativeTurboEngineWithValueHead"]


def _get(tree: Any, path: str, default=None):
    node = tree
    for key in path.split("."):
        if node is None:
            return default
        node = node.get(key) if hasattr(node, "get") else getattr(node, key, None)
    return default if node is None else node


def resolve_turbo_config(engine_config, world: Optional[int] = None):
    """A copy of ``engine_config`` with the ``turbo_config`` tree folded into the engine's own fields."""
    ec = copy.copy(engine_config)
    tree = getattr(engine_config, "turbo_config", None) or {}

    def put(name, value):
        object.__setattr__(ec, name, value)

    for axis in ("tensor_parallel_size", "expert_parallel_size", "expert_fully_shard_parallel_size"):
        if int(_get(tree, f"distributed.{axis}", 1) or 1) > 1:
            raise ValueError(f"turbo_config.distributed.{axis} > 1: tensor and expert parallel training is the "
                             f"strategy=megatron engine in this framework, not an option of fsdp_turbo")
    for key, want in (("param_dtype", "bf16"), ("reduce_dtype", "fp32")):
        got = str(_get(tree, f"distributed.fsdp_plan.{key}", want)).lower().replace("bfloat16", "bf16").replace("float32", "fp32")
        if got != want:
            raise ValueError(f"turbo_config.distributed.fsdp_plan.{key}={got}: this engine keeps {want} here")
    sp_turbo = int(_get(tree, "distributed.ulysses_parallel_size", 1) or 1)
    sp_own = int(getattr(engine_config, "ulysses_sequence_parallel_size", 1) or 1)
    if sp_turbo > 1 and sp_own > 1:
        raise ValueError("Do not enable both turbo_config.distributed.ulysses_parallel_size and "
                         "ulysses_sequence_parallel_size: set one of them")
    if sp_turbo > 1:
        put("ulysses_sequence_parallel_size", sp_turbo)
    fs = int(_get(tree, "distributed.fully_shard_parallel_size", -1) or -1)
    if world is not None and 0 < fs < world and world % fs == 0 and int(getattr(engine_config, "fsdp_size", -1) or -1) <= 0:
        put("fsdp_size", fs)
    raf = _get(tree, "distributed.fsdp_plan.reshard_after_forward")
    if raf is not None:
        put("reshard_after_forward", bool(raf))
    if bool(getattr(engine_config, "offload_policy", False)) or bool(_get(tree, "distributed.fsdp_plan.cpu_offload", False)):
        put("optimizer_offload", True)
    # fully sharded working weights need peers to shard over; hybrid sharding keeps the replicated working copy
    hybrid = 0 < int(getattr(ec, "fsdp_size", -1) or -1) < (world or 1)
    if world is not None and world > 1 and not hybrid and not bool(getattr(engine_config, "forward_only", False)):
        put("zero_stage", 3)
    return ec


class _TurboMixin:
    def initialize(self) -> None:
        if not self._initialized:
            from ....utils.distributed import get_data_parallel_group

            world = dist.get_world_size(get_data_parallel_group()) if dist.is_initialized() else 1
            self.engine_config = resolve_turbo_config(self.engine_config, world)
        super().initialize()


@EngineRegistry.register(model_type="language_model", backend="fsdp_turbo", device=["cuda", "cpu"])
class NativeTurboEngineWithLMHead(_TurboMixin, NativeEngineWithLMHead):
    pass


@EngineRegistry.register(model_type="value_model", backend="fsdp_turbo", device=["cuda", "cpu"])
class NativeTurboEngineWithValueHead(_TurboMixin, NativeEngineWithValueHead):
    pass
