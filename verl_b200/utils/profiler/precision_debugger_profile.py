"""Precision debugger: per-layer tensor statistics (mean, abs-max, norm, NaN / Inf counts) of chosen stages and steps,
written as JSON lines, so that two runs (another parallel layout, another kernel version, another precision) can be
compared layer by layer to find where they start to diverge.

A stage is a named part of the step (``actor_update``, ``actor_compute_log_prob``, ``ref_compute_log_prob``,
``critic_update``, ``compute_values``); the collector attaches to the model's per-layer output hook only while a selected
stage of a selected step runs.
Parity target: ``verl/utils/profiler/precision_debugger_profile.py`` (``PrecisionDebuggerProfiler`` :68 with ``start``
:183, ``stop`` :229, ``annotate`` :239).
"""

from __future__ import annotations

import functools
import json
import os
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

__all__ = ["PrecisionDebuggerToolConfig", "PrecisionDebuggerProfiler", "tensor_stats"]

_STAGES = ("actor_update", "actor_compute_log_prob", "ref_compute_log_prob", "critic_update", "compute_values", "rollout_generate")


@dataclass
class PrecisionDebuggerToolConfig:
    enable: bool = False
    stages: Optional[list] = None      # None = all stages
    steps: Optional[list] = None       # None = every step
    strict: bool = False               # unknown stage names raise instead of being ignored
    save_path: str = "outputs/precision_debug"
    extra: dict = field(default_factory=dict)


def tensor_stats(t: torch.Tensor) -> dict:
    f = t.detach().float()
    finite = torch.isfinite(f)
    g = torch.where(finite, f, torch.zeros_like(f))
    return {"shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", ""), "mean": float(g.mean()) if g.numel() else 0.0,
            "abs_max": float(g.abs().max()) if g.numel() else 0.0, "norm": float(g.norm()),
            "nan": int(torch.isnan(f).sum()), "inf": int(torch.isinf(f).sum())}


class PrecisionDebuggerProfiler:
    def __init__(self, precision_cfg=None, rank: Optional[int] = None, save_path: Optional[str] = None):
        self.config = self._normalize_config(precision_cfg)
        self.rank = int(os.environ.get("RANK", 0)) if rank is None else int(rank)
        self.save_path = save_path or self.config.save_path
        self._stages = self._normalize_stages(self.config.stages)
        self._active: Optional[tuple] = None   # (model, stage, step, records)

    @staticmethod
    def _normalize_config(cfg) -> PrecisionDebuggerToolConfig:
        if cfg is None:
            return PrecisionDebuggerToolConfig()
        if isinstance(cfg, PrecisionDebuggerToolConfig):
            return cfg
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: getattr(cfg, k, d))
        out = PrecisionDebuggerToolConfig()
        for k in ("enable", "stages", "steps", "strict", "save_path"):
            v = get(k, None)
            if v is not None:
                setattr(out, k, list(v) if k in ("stages", "steps") else v)
        return out

    def _normalize_stages(self, stages) -> Optional[set]:
        if stages is None:
            return None
        out = set()
        for s in stages:
            s = str(s).strip().lower()
            if s not in _STAGES:
                if self.config.strict:
                    raise ValueError(f"unknown precision-debugger stage {s!r}; known: {_STAGES}")
                continue
            out.add(s)
        return out

    def _should_collect(self, stage: str, global_step: Optional[int]) -> bool:
        if not self.config.enable:
            return False
        if self._stages is not None and stage not in self._stages:
            return False
        return self.config.steps is None or global_step is None or int(global_step) in set(int(s) for s in self.config.steps)

    # ---- collection
    def start(self, stage: Optional[str] = None, global_step: Optional[int] = None, model=None, **kwargs) -> bool:
        stage = (stage or "").strip().lower()
        if model is None or self._active is not None or not self._should_collect(stage, global_step):
            return False
        records: list[dict] = []
        calls = {}

        def hook(name: str, t: torch.Tensor) -> None:
            k = calls.get(name, 0)
            calls[name] = k + 1
            records.append({"name": name, "call": k, **tensor_stats(t)})

        model.stats_hook = hook
        self._active = (model, stage, global_step, records)
        return True

    def stop(self, started: bool = True) -> Optional[str]:
        if not started or self._active is None:
            return None
        model, stage, step, records = self._active
        model.stats_hook = None
        self._active = None
        os.makedirs(self.save_path, exist_ok=True)
        path = os.path.join(self.save_path, f"{stage}_step{step if step is not None else 'x'}_rank{self.rank}.jsonl")
        with open(path, "w") as f:
            for r in records:
                f.write(json.dumps(r) + "\n")
        return path

    def annotate(self, stage: str, model_attr: str = "model", step_attr: str = "global_step") -> Callable:
        """Decorator for worker / engine methods: collects while the method runs. The model is looked up on ``self`` (dotted
        paths allowed), the step in the keyword arguments or on ``self``."""

        def deco(fn):
            @functools.wraps(fn)
            def wrapped(obj, *args, **kwargs):
                model = obj
                for part in model_attr.split("."):
                    model = getattr(model, part, None)
                    if model is None:
                        break
                step = kwargs.get(step_attr, getattr(obj, step_attr, None))
                started = self.start(stage, step, model)
                try:
                    return fn(obj, *args, **kwargs)
                finally:
                    self.stop(started)

            return wrapped

        return deco
