"""Tinker-style workers: the client owns the training loop and calls three primitives - ``forward_backward`` (may be
called several times to accumulate gradients), ``optimizer_step`` (with per-step optimizer hyper-parameters chosen by the
client: ``lr``, ``betas``, ``eps``, ``weight_decay``) and ``optimizer_zero_grad``. The learning-rate scheduler of the
engine is bypassed.

Parity target: ``verl/workers/engine_workers_tinker.py`` (``OptimStepParams`` :26, ``_apply_optim_step_params`` :63,
``TinkerTrainingWorker`` :110-187, ``TinkerActorRolloutRefWorker`` :189-215).
"""

from __future__ import annotations

from typing import Optional, TypedDict

from ..protocol import DataProto
from ..single_controller.base.decorator import Dispatch, make_nd_compute_dataproto_dispatch_fn, register
from .engine_workers import ActorRolloutRefWorker, TrainingWorker

__all__ = ["OptimStepParams", "TinkerTrainingWorker", "TinkerActorRolloutRefWorker", "apply_optim_step_params"]


class OptimStepParams(TypedDict, total=False):
    lr: float
    eps: float
    betas: tuple
    weight_decay: float


_TYPES = {"lr": (int, float), "eps": (int, float), "weight_decay": (int, float), "betas": (tuple, list)}


def apply_optim_step_params(engine, params: Optional[dict]) -> dict:
    """Validate a step-time override and install it on the engine's optimizer configuration; returns what was replaced so
    that the caller can restore it. Unknown keys and wrongly typed values are errors (nothing is applied then)."""
    if params is None:
        return {}
    if hasattr(params, "to_dict"):
        params = params.to_dict()
    if not isinstance(params, dict):
        raise TypeError(f"optim_step_params must be a dict, got {type(params)}")
    params = {k: v for k, v in params.items() if v is not None}
    for k, v in params.items():
        if k not in _TYPES:
            raise ValueError(f"optimizer does not support optim_step_params key: {k!r}")
        if not isinstance(v, _TYPES[k]) or isinstance(v, bool):
            raise TypeError(f"optim_step_params type mismatch: {k!r} got {type(v).__name__}")
    oc = engine.optimizer_config
    old = {}
    for k, v in params.items():
        old[k] = getattr(oc, k)
        object.__setattr__(oc, k, tuple(v) if k == "betas" else float(v))
    if "lr" in params:
        engine.lr_override = float(params["lr"])
    return old


class _TinkerOps:
    """Mixed into both workers; ``_tinker_engine`` names the engine that trains."""

    def _engine(self):
        return getattr(self, "actor", None) or getattr(self, "engine")

    def _loss(self):
        return getattr(self, "actor_loss", None) or getattr(self, "loss_fn")

    def _zero(self) -> None:
        self._engine().optimizer_zero_grad()

    def _fwd_bwd(self, data: DataProto) -> DataProto:
        eng = self._engine()
        d = {k: v for k, v in data.batch.items()}
        d.update(data.meta_info)
        out = eng.forward_backward_batch(d, self._loss(), forward_only=False)
        metrics = dict(out.get("metrics", {}))
        if "loss" in out:
            metrics["loss"] = float(out["loss"].detach())
        tensors = {k: v for k, v in out.get("model_output", {}).items() if hasattr(v, "shape") and v.dim() >= 1 and v.shape[0] == len(data)}
        res = DataProto.from_dict(tensors=tensors) if tensors else DataProto(meta_info={})
        res.meta_info["metrics"] = metrics
        return res

    def _step(self, optim_step_params: Optional[dict]) -> dict:
        eng = self._engine()
        old = apply_optim_step_params(eng, optim_step_params)
        try:
            norm = eng.optimizer_step()
        finally:
            for k, v in old.items():
                object.__setattr__(eng.optimizer_config, k, v)
            eng.lr_override = None
        return {"grad_norm": float(norm), "lr": float((optim_step_params or {}).get("lr", 0.0) or 0.0)}


class TinkerTrainingWorker(TrainingWorker, _TinkerOps):
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def optimizer_zero_grad(self) -> None:
        self._zero()

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"))
    def forward_backward(self, data: DataProto) -> DataProto:
        return self._fwd_bwd(data)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def optimizer_step(self, optim_step_params: Optional[dict] = None) -> dict:
        return self._step(optim_step_params)


class TinkerActorRolloutRefWorker(ActorRolloutRefWorker, _TinkerOps):
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def optimizer_zero_grad(self) -> None:
        self._zero()

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"))
    def forward_backward(self, data: DataProto) -> DataProto:
        return self._fwd_bwd(self._dev(data))

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def optimizer_step(self, optim_step_params: Optional[dict] = None) -> dict:
        out = self._step(optim_step_params)
        self.update_weights()
        return out
