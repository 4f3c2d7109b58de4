"""Backend names of the reference that have no runtime of their own here, translated onto the two engines that exist.

The reference wraps four more training runtimes (VeOmni, TorchTitan, NeMo-Automodel, MindSpeed). None of them is a
B200 design decision: each is a way to get sharded data parallelism, optionally with tensor / pipeline / context /
expert parallelism, from another library. A user who selects one of those names keeps the *layout* they configured:
``translate`` reads the backend's own option names and returns the engine (``native``: sharded data parallel with Ulysses
/ context parallelism; ``mp``: tensor x pipeline x expert x context parallel) and a config for it with the same parallel
sizes, sharding mode, offload and recomputation settings. Options that only select an implementation inside the foreign
runtime (attention / MoE kernels, compile switches, init device) have no counterpart and are dropped, which the one warning
per backend says.

Parity target: ``verl/workers/engine/{veomni,torchtitan,automodel,mindspeed}/transformer_impl.py`` (the layouts they build
from ``verl/workers/config/engine.py:308-650``).
"""

from __future__ import annotations

import warnings
from dataclasses import fields
from typing import Any

__all__ = ["FOREIGN_BACKENDS", "translate"]

FOREIGN_BACKENDS = ("veomni", "torchtitan", "automodel", "mindspeed")
_warned: set = set()


def _common(src: Any) -> dict:
    """Fields every engine config shares (micro-batching, offload, seeds, ...), copied by name."""
    from ..config import EngineConfig

    return {f.name: getattr(src, f.name) for f in fields(EngineConfig) if f.name not in ("strategy", "_target_") and hasattr(src, f.name)}


def _i(src: Any, *names: str, default: int = 1) -> int:
    """The first of ``names`` that is set to something other than the default (synonyms across backends)."""
    for n in names:
        v = getattr(src, n, None)
        if v is not None and int(v) != default:
            return int(v)
    return default


def translate(backend: str, engine_config: Any):
    """``(engine name, engine config)`` that reproduces the layout ``engine_config`` asks of ``backend``."""
    from ..config import FSDPEngineConfig, McoreEngineConfig

    if backend not in FOREIGN_BACKENDS:
        return backend, engine_config
    src = engine_config
    if backend == "mindspeed" or isinstance(src, McoreEngineConfig):
        target, cfg = "mp", src           # MindSpeed is Megatron's option tree on another accelerator: same layout
    else:
        tp = _i(src, "tensor_parallel_size", "tp_size")
        pp = _i(src, "pipeline_parallel_size", "pp_size")
        ep = _i(src, "expert_parallel_size", "ep_size")
        cp = _i(src, "context_parallel_size", "cp_size")
        etp = _i(src, "expert_tensor_parallel_size")
        sp = _i(src, "ulysses_parallel_size", "ulysses_sequence_parallel_size")
        shard = _i(src, "data_parallel_shard_size", "fsdp_size", default=-1)
        full_shard = bool(getattr(src, "enable_full_shard", False)) or str(getattr(src, "reshard_after_forward", "default")) == "always"
        offload = bool(getattr(src, "enable_fsdp_offload", False)) or bool(getattr(src, "offload_policy", False))
        ckpt = getattr(src, "activation_checkpoint", None)
        recompute = bool(getattr(src, "activation_checkpointing", getattr(src, "enable_gradient_checkpointing", True))) \
            if ckpt is None else str(ckpt) != "none"
        base = _common(src)
        if offload:
            base["optimizer_offload"] = True
        if tp * pp * ep > 1:
            if sp > 1:
                raise ValueError(f"{backend}: Ulysses sequence parallelism together with tensor / pipeline / expert parallelism "
                                 f"is not a layout of this framework; use context_parallel_size")
            cfg = McoreEngineConfig(**base, tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp,
                                    expert_model_parallel_size=ep, context_parallel_size=cp,
                                    expert_tensor_parallel_size=etp if etp > 1 else None,
                                    sequence_parallel=bool(getattr(src, "sequence_parallel", tp > 1)),
                                    enable_gradient_checkpointing=recompute)
            target = "mp"
        else:
            cfg = FSDPEngineConfig(**base, fsdp_size=shard, ulysses_sequence_parallel_size=sp, context_parallel_size=cp,
                                   zero_stage=3 if full_shard else 2, enable_gradient_checkpointing=recompute,
                                   model_dtype=str(getattr(src, "model_dtype", "fp32")))
            target = "native"
    if backend not in _warned:
        _warned.add(backend)
        warnings.warn(f"engine backend '{backend}' runs on this framework's '{target}' engine "
                      f"({'sharded data-parallel' if target == 'native' else 'tensor x pipeline x expert parallel'}) with the "
                      f"parallel sizes, sharding, offload and recomputation settings it was configured with; options that select "
                      f"kernels or compilation inside {backend} itself have no effect", stacklevel=3)
    return target, cfg
