"""Dump intermediate tensors of a run (for comparing two implementations step by step) to a directory, local or remote,
without blocking the training loop: serialisation happens on the caller, the copy on a background thread.

Enabled by ``VERL_ENABLE_TRACKER=1`` with ``VERL_TRACKER_HDFS_DIR`` naming the destination.
Parity target: ``verl/utils/debug/trajectory_tracker.py`` (``TrajectoryTracker`` :51, ``dump_data`` :69,
``get_trajectory_tracker`` :79).
"""

from __future__ import annotations

import io
import os
import tempfile
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Optional

import torch

from .. import hdfs_io

__all__ = ["TrajectoryTracker", "dump_data", "get_trajectory_tracker"]


def save_to_hdfs(data: io.BytesIO, name: str, hdfs_dir: str, verbose: bool) -> str:
    dst = os.path.join(hdfs_dir, f"{name}.pth")
    with tempfile.NamedTemporaryFile(suffix=".pth", delete=False) as f:
        f.write(data.getbuffer())
        tmp = f.name
    try:
        hdfs_io.makedirs(hdfs_dir, exist_ok=True)
        if not hdfs_io.copy(tmp, dst):
            raise IOError(f"could not write {dst}")
        if verbose:
            print(f"saved {name} to {dst}")
    finally:
        os.remove(tmp)
    return dst


class TrajectoryTracker:
    def __init__(self, hdfs_dir: str, verbose: bool = False) -> None:
        self.hdfs_dir, self.verbose = hdfs_dir, verbose
        self._pool = ThreadPoolExecutor(max_workers=1)
        self._pending: list[Future] = []

    def dump(self, data: io.BytesIO, name: str) -> None:
        self._pending.append(self._pool.submit(save_to_hdfs, data, name, self.hdfs_dir, self.verbose))

    def wait_for_hdfs(self) -> list[str]:
        done = [f.result() for f in self._pending]
        self._pending.clear()
        return done


_TRACKER: Optional[TrajectoryTracker] = None


def get_trajectory_tracker() -> Optional[TrajectoryTracker]:
    global _TRACKER
    if _TRACKER is None and os.environ.get("VERL_ENABLE_TRACKER", "0") == "1":
        _TRACKER = TrajectoryTracker(os.environ.get("VERL_TRACKER_HDFS_DIR", os.path.join(tempfile.gettempdir(), "verl-tracker")),
                                     verbose=os.environ.get("VERL_TRACKER_VERBOSE", "0") == "1")
    return _TRACKER


def dump_data(data, name: str) -> None:
    """No-op unless the tracker is enabled."""
    tracker = get_trajectory_tracker()
    if tracker is None:
        return
    buf = io.BytesIO()
    torch.save(data, buf)
    tracker.dump(buf, name)
