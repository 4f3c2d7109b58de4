"""Checkpoint manager of the tensor/pipeline-parallel engine: one ``mp_rank_{tp:02d}_{pp:03d}/`` directory per model
parallel rank (``model.pt`` with HF-named local tensors, ``optim.pt`` per data-parallel shard owner), which
``verl_b200.model_merger`` (backend ``megatron``) folds back into one HuggingFace model.

Parity target: ``verl/utils/checkpoint/megatron_checkpoint_manager.py`` (dist-checkpoint layout, HF export, rotation).
"""

from __future__ import annotations

import os
from typing import Optional

import torch

from .checkpoint_manager import BaseCheckpointManager

__all__ = ["MegatronCheckpointManager"]


class MegatronCheckpointManager(BaseCheckpointManager):
    def __init__(self, engine, tp_rank: int, pp_rank: int, dp_rank: int, processing_class=None, checkpoint_config=None):
        super().__init__(model=engine, processing_class=processing_class, checkpoint_config=checkpoint_config)
        self.engine, self.tp_rank, self.pp_rank, self.dp_rank = engine, tp_rank, pp_rank, dp_rank

    def _dir(self, root: str) -> str:
        return os.path.join(root, f"mp_rank_{self.tp_rank:02d}_{self.pp_rank:03d}")

    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None) -> None:
        d = self._dir(local_path)
        os.makedirs(d, exist_ok=True)
        if self.dp_rank == 0 and self.should_save_model:
            torch.save({k: v.detach().cpu() for k, v in self.engine.local_named_tensors()}, os.path.join(d, "model.pt"))
        if self.should_save_optimizer and hasattr(self.engine, "optimizer_state"):
            torch.save(self.engine.optimizer_state(), os.path.join(d, f"optim_dp{self.dp_rank}.pt"))
        if self.should_save_extra:
            torch.save({"rng": self.get_rng_state(), "global_step": global_step}, os.path.join(d, f"extra_dp{self.dp_rank}.pt"))
        self.register_checkpoint(local_path, max_ckpt_to_keep)

    def load_checkpoint(self, local_path: Optional[str], hdfs_path: Optional[str] = None, del_local_after_load: bool = False) -> None:
        if local_path is None:
            return
        d = self._dir(local_path)
        mp = os.path.join(d, "model.pt")
        if self.should_load_model and os.path.exists(mp):
            self.engine.load_local_named_tensors(torch.load(mp, map_location="cpu", weights_only=False))
        op = os.path.join(d, f"optim_dp{self.dp_rank}.pt")
        if self.should_load_optimizer and os.path.exists(op) and hasattr(self.engine, "load_optimizer_state"):
            self.engine.load_optimizer_state(torch.load(op, map_location="cpu", weights_only=False))
        ep = os.path.join(d, f"extra_dp{self.dp_rank}.pt")
        if self.should_load_extra and os.path.exists(ep):
            self.load_rng_state(torch.load(ep, map_location="cpu", weights_only=False)["rng"])
