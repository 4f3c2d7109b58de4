"""Device-memory housekeeping and diagnostics: cache trimming between training and rollout phases, usage reports, and
allocator-history snapshots that can be opened in PyTorch's memory visualiser.

Parity target: ``verl/utils/memory_utils.py`` (``aggressive_empty_cache`` :31, ``reset_memory_stats`` :77,
``get_memory_info`` :85, ``log_memory_usage`` :103, ``optimize_memory_for_inference`` :118,
``optimize_memory_for_training`` :132, ``enable_memory_visualize`` :146, ``clear_memory_history`` :241,
``MemorySnapshotSampler`` :253).
"""

from __future__ import annotations

import gc
import logging
import os
import time
from typing import Optional

import torch

logger = logging.getLogger(__name__)

__all__ = ["aggressive_empty_cache", "reset_memory_stats", "get_memory_info", "log_memory_usage", "optimize_memory_for_inference",
           "optimize_memory_for_training", "enable_memory_visualize", "clear_memory_history", "MemorySnapshotSampler"]


def _cuda() -> bool:
    return torch.cuda.is_available()


def aggressive_empty_cache(force_sync: bool = True, max_retries: int = 3) -> None:
    """Collect garbage and return cached blocks to the driver, repeating while that still frees a noticeable amount
    (objects released by one collection can release tensors that the next pass frees)."""
    if not _cuda():
        gc.collect()
        return
    for _ in range(max_retries):
        before = torch.cuda.memory_reserved()
        gc.collect()
        torch.cuda.empty_cache()
        if force_sync:
            torch.cuda.synchronize()
        if before - torch.cuda.memory_reserved() < (1 << 30):
            break


def reset_memory_stats() -> None:
    if _cuda():
        torch.cuda.reset_peak_memory_stats()
        torch.cuda.reset_accumulated_memory_stats()


def get_memory_info() -> dict:
    """GiB figures of the current device; empty without a GPU."""
    if not _cuda():
        return {}
    free, total = torch.cuda.mem_get_info()
    g = 1 << 30
    return {"allocated_gb": torch.cuda.memory_allocated() / g, "reserved_gb": torch.cuda.memory_reserved() / g,
            "max_allocated_gb": torch.cuda.max_memory_allocated() / g, "max_reserved_gb": torch.cuda.max_memory_reserved() / g,
            "free_gb": free / g, "total_gb": total / g}


def log_memory_usage(stage: str = "current") -> None:
    info = get_memory_info()
    if info:
        logger.info("memory at %s: %s", stage, ", ".join(f"{k}={v:.2f}" for k, v in info.items()))


def optimize_memory_for_inference() -> None:
    """Before a rollout phase: nothing of the training step's transient memory should stay cached."""
    aggressive_empty_cache(force_sync=True)


def optimize_memory_for_training() -> None:
    aggressive_empty_cache(force_sync=False)


def enable_memory_visualize(trace_alloc_max_entries: int = 200_000, stack_depth: int = 32, context: str = "all",
                            stacks: str = "all", devices=None, record_context: bool = True) -> None:
    """Start recording allocator history (allocation stack traces) for later snapshots."""
    if not _cuda():
        logger.warning("memory history needs a GPU; ignored")
        return
    torch.cuda.memory._record_memory_history(enabled="all", context=context if record_context else None, stacks=stacks,
                                             max_entries=trace_alloc_max_entries)


def clear_memory_history(trace_alloc_max_entries: int = 200_000, stack_depth: int = 32) -> None:
    """Drop what was recorded so far and keep recording."""
    if _cuda():
        torch.cuda.memory._record_memory_history(enabled=None)
        enable_memory_visualize(trace_alloc_max_entries, stack_depth)


class MemorySnapshotSampler:
    """Writes allocator snapshots (``.pickle``, loadable at pytorch.org/memory_viz) named by tag, rank and time."""

    def __init__(self, out_dir: str = "./mem_snapshots", tag: str = "periodic"):
        self.out_dir, self.tag = out_dir, tag

    def dump_memory_snapshot(self, out_dir: Optional[str] = None, tag: Optional[str] = None, sub_dir: Optional[str] = None) -> Optional[str]:
        if not _cuda():
            return None
        d = os.path.join(out_dir or self.out_dir, sub_dir) if sub_dir else (out_dir or self.out_dir)
        os.makedirs(d, exist_ok=True)
        rank = int(os.environ.get("RANK", "0"))
        path = os.path.join(d, f"{tag or self.tag}_rank{rank}_{time.strftime('%Y%m%d-%H%M%S')}.pickle")
        torch.cuda.memory._dump_snapshot(path)
        return path
