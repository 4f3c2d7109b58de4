"""Distributed profiler front-end: NVTX ranges + cudaProfilerStart/Stop (for nsys/ncu), torch.profiler traces and
allocator memory snapshots, selected per rank and per step.

Parity target: ``verl/utils/profiler/profile.py`` (``DistProfiler`` :88-379, ``DistProfilerExtension`` :428-463) and the
tool back-ends ``nvtx_profile.py``, ``torch_profile.py``, ``torch_memory_profile.py``.
"""

from __future__ import annotations

import functools
import os
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from ...base_config import BaseConfig
from ...single_controller.base.decorator import Dispatch, register
from ..device import get_device_name

__all__ = ["ProfilerConfig", "DistProfiler", "DistProfilerExtension", "mark_start_range", "mark_end_range", "mark_annotate"]


@dataclass
class ProfilerConfig(BaseConfig):
    tool: Optional[str] = None  # nsys | torch | torch_memory | None
    enable: bool = False
    all_ranks: bool = False
    ranks: list = field(default_factory=list)
    save_path: str = "outputs/profile"
    steps: Optional[list] = None
    discrete: bool = False
    tool_config: dict = field(default_factory=dict)
    profile_continuous_steps: bool = False


def mark_start_range(message: Optional[str] = None, color: Optional[str] = None, domain=None, category=None):
    if get_device_name() == "cuda":
        torch.cuda.nvtx.range_push(message or "range")
    return message


def mark_end_range(range_id=None) -> None:
    if get_device_name() == "cuda":
        torch.cuda.nvtx.range_pop()


def mark_annotate(message: Optional[str] = None, color: Optional[str] = None, domain=None, category=None) -> Callable:
    def deco(fn):
        @functools.wraps(fn)
        def wrapped(*a, **k):
            mark_start_range(message or fn.__name__)
            try:
                return fn(*a, **k)
            finally:
                mark_end_range()

        return wrapped

    return deco


class DistProfiler:
    """Start/stop/step a profiling tool on the ranks selected by the config."""

    def __init__(self, rank: int, config: Optional[ProfilerConfig] = None, tool_config=None, **kwargs):
        self.rank = rank
        self.config = config or ProfilerConfig()
        self.tool = self.config.tool if self.config.enable else None
        self.active = False
        self._prof = None
        self._precision, self._precision_started = None, False
        self._step = 0

    def _selected(self) -> bool:
        return bool(self.tool) and (self.config.all_ranks or self.rank in list(self.config.ranks or []))

    def start(self, **kwargs) -> None:
        if not self._selected() or self.active:
            return
        self.active = True
        if self.tool == "nsys" and get_device_name() == "cuda":
            torch.cuda.cudart().cudaProfilerStart()
        elif self.tool == "torch":
            acts = [torch.profiler.ProfilerActivity.CPU]
            if get_device_name() == "cuda":
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._prof = torch.profiler.profile(activities=acts, record_shapes=True,
                                                with_stack=bool(self.config.tool_config.get("with_stack", False)))
            self._prof.__enter__()
        elif self.tool == "torch_memory" and get_device_name() == "cuda":
            torch.cuda.memory._record_memory_history(max_entries=int(self.config.tool_config.get("trace_alloc_max_entries", 100000)))
        elif self.tool == "precision_debugger":
            from .precision_debugger_profile import PrecisionDebuggerProfiler

            if self._precision is None:
                self._precision = PrecisionDebuggerProfiler(dict(self.config.tool_config or {}, enable=True), rank=self.rank,
                                                            save_path=self.config.save_path)
            self._precision_started = self._precision.start(kwargs.get("stage", "actor_update"), kwargs.get("global_step", self._step),
                                                            kwargs.get("model"))

    def stop(self) -> None:
        if not self.active:
            return
        self.active = False
        os.makedirs(self.config.save_path, exist_ok=True)
        if self.tool == "nsys" and get_device_name() == "cuda":
            torch.cuda.cudart().cudaProfilerStop()
        elif self.tool == "torch" and self._prof is not None:
            self._prof.__exit__(None, None, None)
            self._prof.export_chrome_trace(os.path.join(self.config.save_path, f"trace_rank{self.rank}_step{self._step}.json"))
            self._prof = None
        elif self.tool == "precision_debugger" and self._precision is not None:
            self._precision.stop(self._precision_started)
        elif self.tool == "torch_memory" and get_device_name() == "cuda":
            torch.cuda.memory._dump_snapshot(os.path.join(self.config.save_path, f"memory_rank{self.rank}_step{self._step}.pickle"))
            torch.cuda.memory._record_memory_history(enabled=None)

    def step(self) -> None:
        self._step += 1
        if self._prof is not None:
            self._prof.step()

    @staticmethod
    def annotate(message: Optional[str] = None, color: Optional[str] = None, role: Optional[str] = None, **kwargs) -> Callable:
        return mark_annotate(message, color)


class DistProfilerExtension:
    """Mixin giving every worker ``start_profile`` / ``stop_profile`` / ``step_profile`` RPCs."""

    def __init__(self, profiler: Optional[DistProfiler] = None):
        rank = int(os.environ.get("RANK", 0))
        if profiler is None or isinstance(profiler, (dict, ProfilerConfig)):
            cfg = profiler if isinstance(profiler, ProfilerConfig) else (ProfilerConfig.from_dict(profiler) if profiler else None)
            profiler = DistProfiler(rank, cfg)
        self.profiler = profiler

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def start_profile(self, **kwargs) -> None:
        self.profiler.start(**kwargs)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def stop_profile(self) -> None:
        self.profiler.stop()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def step_profile(self) -> None:
        self.profiler.step()
