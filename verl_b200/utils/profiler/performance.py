"""Timers and memory logging. Parity target: ``verl/utils/profiler/performance.py`` (:63-256)."""

from __future__ import annotations

import logging
import time
from contextlib import contextmanager
from typing import Optional

import torch
import torch.distributed as dist

from ..device import get_device_name

__all__ = ["log_gpu_memory_usage", "GPUMemoryLogger", "simple_timer", "marked_timer", "reduce_timing", "gather_timing",
           "DeviceTimer"]


def _mem():
    if get_device_name() != "cuda":
        return 0.0, 0.0, 0.0, 0.0
    free, total = torch.cuda.mem_get_info()
    g = 1024**3
    return torch.cuda.memory_allocated() / g, torch.cuda.memory_reserved() / g, (total - free) / g, total / g


def log_gpu_memory_usage(head: str, logger: Optional[logging.Logger] = None, level=logging.DEBUG, rank: int = 0) -> None:
    if dist.is_initialized() and rank is not None and dist.get_rank() != rank:
        return
    a, r, u, t = _mem()
    msg = f"{head}, memory allocated (GB): {a:.2f}, memory reserved (GB): {r:.2f}, device memory used/total (GB): {u:.2f}/{t:.2f}"
    (logger.log(level, msg) if logger is not None else print(msg))


class GPUMemoryLogger:
    """Decorator logging device memory before and after a method call."""

    def __init__(self, role: str, logger=None, level=logging.DEBUG, log_only_rank_0: bool = True):
        self.role, self.logger, self.level, self.rank0 = role, logger, level, log_only_rank_0

    def __call__(self, fn):
        def wrapped(*a, **k):
            log_gpu_memory_usage(f"[{self.role}] before {fn.__name__}", self.logger, self.level, 0 if self.rank0 else None)
            out = fn(*a, **k)
            log_gpu_memory_usage(f"[{self.role}] after {fn.__name__}", self.logger, self.level, 0 if self.rank0 else None)
            return out

        return wrapped


@contextmanager
def simple_timer(name: str, timing_raw: dict):
    t0 = time.perf_counter()
    yield
    timing_raw[name] = timing_raw.get(name, 0.0) + time.perf_counter() - t0


@contextmanager
def marked_timer(name: str, timing_raw: dict, color: str = None, **kwargs):
    """Wall-clock timer that also opens an NVTX range when a CUDA device is present."""
    pushed = False
    if get_device_name() == "cuda":
        try:
            torch.cuda.nvtx.range_push(name)
            pushed = True
        except Exception:
            pushed = False
    t0 = time.perf_counter()
    try:
        yield
    finally:
        timing_raw[name] = timing_raw.get(name, 0.0) + time.perf_counter() - t0
        if pushed:
            torch.cuda.nvtx.range_pop()


class DeviceTimer:
    """CUDA-event timer on the current stream (host wall-clock on CPU). ``elapsed_ms`` synchronises."""

    def __init__(self):
        self.cuda = get_device_name() == "cuda"
        self._spans: dict[str, list] = {}

    @contextmanager
    def span(self, name: str):
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            yield
            b.record()
            self._spans.setdefault(name, []).append((a, b))
        else:
            t0 = time.perf_counter()
            yield
            self._spans.setdefault(name, []).append((t0, time.perf_counter()))

    def elapsed_ms(self) -> dict[str, float]:
        if self.cuda:
            torch.cuda.synchronize()
            return {k: sum(a.elapsed_time(b) for a, b in v) for k, v in self._spans.items()}
        return {k: sum((b - a) * 1e3 for a, b in v) for k, v in self._spans.items()}


def reduce_timing(timing_raw: dict, reduce_op=None) -> dict:
    """All-reduce (mean by default) every timing value across ranks."""
    if not dist.is_initialized() or not timing_raw:
        return timing_raw
    keys = sorted(timing_raw)
    dev = "cuda" if get_device_name() == "cuda" else "cpu"
    t = torch.tensor([float(timing_raw[k]) for k in keys], dtype=torch.float32, device=dev)
    op = reduce_op or dist.ReduceOp.SUM
    dist.all_reduce(t, op=op)
    if reduce_op is None:
        t /= dist.get_world_size()
    return {k: float(v) for k, v in zip(keys, t.tolist())}


def gather_timing(timing_raw: dict) -> list[dict]:
    if not dist.is_initialized():
        return [timing_raw]
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, timing_raw)
    return out
