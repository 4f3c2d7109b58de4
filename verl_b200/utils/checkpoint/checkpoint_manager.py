"""Checkpoint bookkeeping: latest-step tracking, rotation, RNG state, preemption-aware saving.

Parity target: ``verl/utils/checkpoint/checkpoint_manager.py`` (``BaseCheckpointManager`` :29-219,
``find_latest_ckpt_path`` :222-259, ``should_save_ckpt_esi`` :262-293).
"""

from __future__ import annotations

import os
import random
import re
import shutil
import time
from typing import Optional

import numpy as np
import torch

__all__ = ["BaseCheckpointManager", "find_latest_ckpt_path", "get_checkpoint_tracker_filename", "should_save_ckpt_esi",
           "rotate_checkpoints"]


def get_checkpoint_tracker_filename(root_path: str) -> str:
    return os.path.join(root_path, "latest_checkpointed_iteration.txt")


def find_latest_ckpt_path(path: Optional[str], directory_format: str = "global_step_{}") -> Optional[str]:
    """The checkpoint folder named by the tracker file under ``path`` (None when absent or stale)."""
    if path is None:
        return None
    tracker = get_checkpoint_tracker_filename(path)
    if not os.path.exists(tracker):
        return None
    with open(tracker) as f:
        it = int(f.read().strip())
    ckpt = os.path.join(path, directory_format.format(it))
    if not os.path.exists(ckpt):
        print(f"Checkpoint does not exist: {ckpt}")
        return None
    print(f"Found checkpoint: {ckpt}")
    return ckpt


def rotate_checkpoints(root: str, keep: int, directory_format: str = r"global_step_(\d+)") -> list[str]:
    """Delete the oldest ``global_step_N`` folders so that at most ``keep`` remain; returns what was removed."""
    steps = []
    for name in os.listdir(root):
        m = re.fullmatch(directory_format, name)
        if m:
            steps.append((int(m.group(1)), os.path.join(root, name)))
    steps.sort()
    removed = []
    while keep > 0 and len(steps) > keep:
        _, p = steps.pop(0)
        shutil.rmtree(p, ignore_errors=True)
        removed.append(p)
    return removed


def should_save_ckpt_esi(max_steps_duration: float, save_ckpt_duration: float = 60, redundant_time: float = 0) -> bool:
    """True when a capacity-block / spot expiry (env ``*_EXPIRATION_TIMESTAMP``) would hit before another step and a
    checkpoint could complete."""
    exp = None
    for key in ("MLP_CURRENT_CAPACITY_BLOCK_EXPIRATION_TIMESTAMP", "SAGEMAKER_CURRENT_CAPACITY_BLOCK_EXPIRATION_TIMESTAMP",
                "VERL_CAPACITY_EXPIRATION_TIMESTAMP"):
        if os.getenv(key):
            exp = float(os.getenv(key))
            break
    if exp is None:
        return False
    remaining = exp - time.time()
    return 0 < remaining <= max_steps_duration + save_ckpt_duration + redundant_time


class BaseCheckpointManager:
    """Common state for engine checkpoint managers (content flags, rotation list, RNG capture)."""

    def __init__(self, model=None, optimizer=None, lr_scheduler=None, processing_class=None, checkpoint_config=None):
        self.model, self.optimizer, self.lr_scheduler = model, optimizer, lr_scheduler
        self.processing_class = processing_class
        self.checkpoint_config = checkpoint_config
        self.previous_global_step = None
        self.previous_saved_paths: list[str] = []
        self.rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else 0
        self.world_size = torch.distributed.get_world_size() if torch.distributed.is_initialized() else 1

    def _flags(self, which: str) -> list:
        d = self.checkpoint_config
        v = None
        if d is not None:  # a mapping (config tree) or an object with attributes (dataclass)
            v = d.get(which) if hasattr(d, "get") else getattr(d, which, None)
        v = v or ["model", "optimizer", "extra"]
        return list(v)

    @property
    def should_save_model(self) -> bool:
        return "model" in self._flags("save_contents")

    @property
    def should_save_optimizer(self) -> bool:
        return "optimizer" in self._flags("save_contents")

    @property
    def should_save_extra(self) -> bool:
        return "extra" in self._flags("save_contents")

    @property
    def should_save_hf_model(self) -> bool:
        return "hf_model" in self._flags("save_contents")

    @property
    def should_load_model(self) -> bool:
        return "model" in self._flags("load_contents")

    @property
    def should_load_optimizer(self) -> bool:
        return "optimizer" in self._flags("load_contents")

    @property
    def should_load_extra(self) -> bool:
        return "extra" in self._flags("load_contents")

    def load_checkpoint(self, local_path: str, hdfs_path: str = None, del_local_after_load: bool = False):
        raise NotImplementedError

    def save_checkpoint(self, local_path: str, hdfs_path: str = None, global_step: int = 0, max_ckpt_to_keep: int = None):
        raise NotImplementedError

    @staticmethod
    def checkpath(local_path: str, hdfs_path: str):
        assert local_path is not None or hdfs_path is not None, "local_path and hdfs_path cannot be both None"
        return local_path is not None, local_path if local_path is not None else hdfs_path

    def remove_previous_save_local_path(self, path) -> None:
        for p in ([path] if isinstance(path, str) else path):
            p = os.path.abspath(p)
            if os.path.exists(p):
                shutil.rmtree(p, ignore_errors=True)

    def ensure_checkpoint_capacity(self, max_ckpt_to_keep: Optional[int]) -> None:
        if isinstance(max_ckpt_to_keep, int) and max_ckpt_to_keep > 0 and len(self.previous_saved_paths) >= max_ckpt_to_keep:
            n = len(self.previous_saved_paths) - max_ckpt_to_keep + 1
            self.remove_previous_save_local_path(self.previous_saved_paths[:n])
            self.previous_saved_paths = self.previous_saved_paths[n:]

    def register_checkpoint(self, path: str, max_ckpt_to_keep: Optional[int]) -> None:
        self.previous_saved_paths.append(path)

    @staticmethod
    def get_rng_state() -> dict:
        st = {"cpu": torch.get_rng_state(), "numpy": np.random.get_state(), "random": random.getstate()}
        if torch.cuda.is_available():
            st["cuda"] = torch.cuda.get_rng_state()
        return st

    @staticmethod
    def load_rng_state(st: dict) -> None:
        torch.set_rng_state(st["cpu"])
        np.random.set_state(st["numpy"])
        random.setstate(st["random"])
        if torch.cuda.is_available() and "cuda" in st:
            torch.cuda.set_rng_state(st["cuda"])
