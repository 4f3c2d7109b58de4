"""Training-engine interface and registry.

An engine owns one model replica/shard set with its optimizer and exposes the operations the worker roles
need: micro-batched forward/backward with a pluggable loss, optimizer and LR-scheduler steps, weight export
for the rollout side, host offload and checkpointing.

Parity target: ``verl/workers/engine/base.py`` (``BaseEngine`` :30-298, ``BaseEngineCtx`` :300-336,
``EngineRegistry`` :339-445).
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Callable, Generator, Optional

import torch

__all__ = ["BaseEngine", "BaseEngineCtx", "EngineRegistry"]


class BaseEngine(ABC):
    """Abstract engine; concrete engines register themselves in :class:`EngineRegistry`."""

    def initialize(self) -> None:
        raise NotImplementedError

    # -- modes ---------------------------------------------------------------------------------
    def train_mode(self, **kwargs) -> "BaseEngineCtx":
        return BaseEngineCtx(self, "train", **kwargs)

    def eval_mode(self, **kwargs) -> "BaseEngineCtx":
        return BaseEngineCtx(self, "eval", **kwargs)

    # -- compute -------------------------------------------------------------------------------
    @abstractmethod
    def forward_backward_batch(self, data, loss_function: Optional[Callable], forward_only: bool = False) -> dict:
        ...

    def optimizer_zero_grad(self) -> None:
        raise NotImplementedError

    def optimizer_step(self) -> float:
        raise NotImplementedError

    def lr_scheduler_step(self) -> float:
        raise NotImplementedError

    def train_batch(self, data, loss_function: Callable) -> dict:
        """zero-grad -> forward/backward over micro-batches -> optimizer step -> scheduler step."""
        self.optimizer_zero_grad()
        out = self.forward_backward_batch(data, loss_function, forward_only=False)
        ev = None
        if torch.cuda.is_available() and getattr(getattr(self, "device", None), "type", "cpu") == "cuda":
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        grad_norm = self.optimizer_step()
        if ev is not None:  # device time of the optimizer step (gradient reduction, clip, update, weight publication)
            ev[1].record()
            ev[1].synchronize()
            self.last_optimizer_step_s = ev[0].elapsed_time(ev[1]) * 1e-3
        lr = self.lr_scheduler_step()
        out.setdefault("metrics", {})
        out["metrics"]["grad_norm"] = grad_norm
        out["metrics"]["lr"] = lr
        return out

    def infer_batch(self, data, loss_function: Optional[Callable] = None) -> dict:
        with torch.no_grad():
            return self.forward_backward_batch(data, loss_function, forward_only=True)

    # -- weights -------------------------------------------------------------------------------
    def get_per_tensor_param(self, **kwargs) -> Generator[tuple[str, torch.Tensor], None, None]:
        raise NotImplementedError

    def get_per_tensor_param_shard(self, **kwargs):
        raise NotImplementedError

    # -- topology ------------------------------------------------------------------------------
    def get_data_parallel_size(self) -> int:
        raise NotImplementedError

    def get_data_parallel_rank(self) -> int:
        raise NotImplementedError

    def get_data_parallel_group(self):
        raise NotImplementedError

    def is_mp_src_rank_with_outputs(self) -> bool:
        return True

    # -- residency / checkpoint ----------------------------------------------------------------
    def to(self, device: str, model: bool = True, optimizer: bool = True, grad: bool = True) -> None:
        raise NotImplementedError

    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None, **kwargs) -> None:
        raise NotImplementedError

    def load_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, del_local_after_load: bool = False,
                        **kwargs) -> None:
        raise NotImplementedError


class BaseEngineCtx:
    """Context manager that makes the engine resident for a phase and offloads it again afterwards."""

    def __init__(self, engine: BaseEngine, mode: str, **kwargs):
        self.engine, self.mode, self.kwargs = engine, mode, kwargs

    def __enter__(self):
        hook = getattr(self.engine, "_enter_mode", None)
        if hook is not None:
            hook(self.mode, **self.kwargs)
        return self.engine

    def __exit__(self, exc_type, exc, tb):
        hook = getattr(self.engine, "_exit_mode", None)
        if hook is not None:
            hook(self.mode, **self.kwargs)
        return False


class EngineRegistry:
    """(model_type, backend, device) -> engine class."""

    _engines: dict[str, dict[str, dict[str, type]]] = {}

    @classmethod
    def register(cls, model_type: str, backend, device="cuda"):
        backends = [backend] if isinstance(backend, str) else list(backend)
        devices = [device] if isinstance(device, str) else list(device)

        def deco(engine_cls):
            for b in backends:
                for d in devices:
                    cls._engines.setdefault(model_type, {}).setdefault(b, {})[d] = engine_cls
            return engine_cls

        return deco

    # backend names of the reference that have no runtime of their own here: ``new`` translates their option names onto
    # one of the two engines (``backends.translate``); a bare class lookup gets the engine their default layout runs on
    ALIASES = {"veomni": "native", "torchtitan": "native", "automodel": "native", "mindspeed": "mp"}

    @classmethod
    def get_engine_cls(cls, model_type: str, backend: str, device: Optional[str] = None):
        from ...utils.device import get_device_name

        device = device or get_device_name()
        if backend not in cls._engines.get(model_type, {}) and backend not in ("megatron", "mp", "mindspeed"):
            from .native import engine  # noqa: F401  (registers the sharded data-parallel engines)
        if backend == "fsdp_turbo" and backend not in cls._engines.get(model_type, {}):
            from .native import turbo  # noqa: F401  (registers the fully sharded, fused configuration of the native engine)
        if backend in ("megatron", "mp", "mindspeed") and backend not in cls._engines.get(model_type, {}):
            from . import mp  # noqa: F401  (registers the tensor x pipeline parallel engines)
        try:
            return cls._engines[model_type][backend][device]
        except KeyError:
            raise ValueError(f"no engine registered for model_type={model_type!r} backend={backend!r} "
                             f"device={device!r}; known: { {m: list(b) for m, b in cls._engines.items()} }") from None

    @classmethod
    def new(cls, model_type: str, backend: str, *args, **kwargs) -> BaseEngine:
        device = kwargs.pop("device", None)
        from .backends import FOREIGN_BACKENDS, translate

        if backend in FOREIGN_BACKENDS:
            args = list(args)
            ec = kwargs.get("engine_config", args[1] if len(args) > 1 else None)
            if ec is not None:
                backend, ec = translate(backend, ec)
                if "engine_config" in kwargs or len(args) < 2:
                    kwargs["engine_config"] = ec
                else:
                    args[1] = ec
        return cls.get_engine_cls(model_type, backend, device)(*args, **kwargs)
