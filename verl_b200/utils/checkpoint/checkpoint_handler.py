"""Trainer-side checkpoint orchestration for SFT-style loops: where to save, when to rotate, how to resume
(``auto`` = latest ``global_step_N`` under the run directory, ``resume_path`` = a given one, ``disable``), including
the dataloader state so that a resumed run continues with the next batch.

Parity target: ``verl/utils/checkpoint/checkpoint_handler.py`` (``OrchestrationMode`` :44, ``CheckpointHandler`` :49-240).
"""

from __future__ import annotations

import os
import re
from enum import Enum
from typing import Optional

import torch

from .checkpoint_manager import find_latest_ckpt_path, rotate_checkpoints

__all__ = ["OrchestrationMode", "CheckpointHandler"]


class OrchestrationMode(Enum):
    SPMD = "spmd"   # every rank runs the handler (torchrun); rank 0 writes the tracker file
    RAY = "ray"     # one controller runs the handler and calls the engines remotely


class CheckpointHandler:
    def __init__(self, engine, train_dataloader=None, rank: int = 0, default_local_dir: str = "checkpoints", max_ckpt_to_keep: Optional[int] = None,
                 default_hdfs_dir: Optional[str] = None, resume_mode: str = "auto", resume_from_path: Optional[str] = None,
                 mode: OrchestrationMode = OrchestrationMode.SPMD):
        self.engine, self.train_dataloader, self.rank = engine, train_dataloader, rank
        self.default_local_dir, self.default_hdfs_dir = default_local_dir, default_hdfs_dir
        self.max_ckpt_to_keep, self.resume_mode, self.resume_from_path, self.mode = max_ckpt_to_keep, resume_mode, resume_from_path, mode

    def save_checkpoint(self, step: int) -> str:
        path = os.path.join(self.default_local_dir, f"global_step_{step}")
        hdfs = os.path.join(self.default_hdfs_dir, f"global_step_{step}") if self.default_hdfs_dir else None
        self.engine.save_checkpoint(local_path=path, hdfs_path=hdfs, global_step=step, max_ckpt_to_keep=self.max_ckpt_to_keep)
        if self.train_dataloader is not None and hasattr(self.train_dataloader, "state_dict"):
            name = "data.pt" if self.mode is OrchestrationMode.RAY else f"data_rank{self.rank}.pt"
            os.makedirs(path, exist_ok=True)
            torch.save(self.train_dataloader.state_dict(), os.path.join(path, name))
        if self.rank == 0:
            with open(os.path.join(self.default_local_dir, "latest_checkpointed_iteration.txt"), "w") as f:
                f.write(str(step))
            if self.max_ckpt_to_keep:
                rotate_checkpoints(self.default_local_dir, int(self.max_ckpt_to_keep))
        return path

    def _determine_resume_path(self) -> Optional[str]:
        if self.resume_mode == "disable":
            return None
        if self.resume_mode == "resume_path":
            assert self.resume_from_path and "global_step_" in self.resume_from_path, "resume_from_path must name a global_step_N directory"
            return self.resume_from_path
        return find_latest_ckpt_path(self.default_local_dir)

    def load_checkpoint(self) -> int:
        """Returns the step to continue from (0 when starting fresh)."""
        path = self._determine_resume_path()
        if not path:
            return 0
        self.engine.load_checkpoint(local_path=path)
        self._load_dataloader_state(path)
        m = re.search(r"global_step_(\d+)", str(path))
        return int(m.group(1)) if m else 0

    def _load_dataloader_state(self, path: str) -> None:
        if self.train_dataloader is None or not hasattr(self.train_dataloader, "load_state_dict"):
            return
        for name in (f"data_rank{self.rank}.pt", "data.pt"):
            p = os.path.join(path, name)
            if os.path.exists(p):
                self.train_dataloader.load_state_dict(torch.load(p, weights_only=False))
                return
