"""Sharded checkpoint manager of the native (FSDP-role) engine: every data-parallel rank writes its slice of the flat
fp32 master weights and optimizer moments as ``model_world_size_{W}_rank_{r}.pt`` / ``optim_…`` / ``extra_state_…``;
rank 0 adds ``fsdp_config.json`` and a ``huggingface/`` directory (config, tokenizer; full weights when
``hf_model`` is among ``save_contents``). Rotation keeps the newest ``max_ckpt_to_keep`` directories.

Parity target: ``verl/utils/checkpoint/fsdp_checkpoint_manager.py`` (file naming :140-260, ``FSDPConfig`` json, HF export).
"""

from __future__ import annotations

import os
from typing import Optional

from .checkpoint_manager import BaseCheckpointManager

__all__ = ["FSDPCheckpointManager"]


class FSDPCheckpointManager(BaseCheckpointManager):
    def __init__(self, engine, processing_class=None, checkpoint_config=None, **kwargs):
        super().__init__(model=engine, optimizer=None, lr_scheduler=None, processing_class=processing_class,
                         checkpoint_config=checkpoint_config if checkpoint_config is not None else getattr(engine, "checkpoint_config", None))
        self.engine = engine
        self.rank, self.world_size = engine.rank, engine.world

    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None) -> None:
        if local_path is None:
            return
        self.previous_global_step = global_step
        if self.rank == 0:
            self.ensure_checkpoint_capacity(max_ckpt_to_keep)
        self.engine.save_checkpoint(local_path, hdfs_path, global_step, max_ckpt_to_keep)
        if self.rank == 0 and self.processing_class is not None and hasattr(self.processing_class, "save_pretrained"):
            self.processing_class.save_pretrained(os.path.join(local_path, "huggingface"))
        self.register_checkpoint(local_path, max_ckpt_to_keep)

    def load_checkpoint(self, local_path: Optional[str], hdfs_path: Optional[str] = None, del_local_after_load: bool = False) -> None:
        if local_path is None:
            return
        self.engine.load_checkpoint(local_path, hdfs_path, del_local_after_load)
        if del_local_after_load and self.rank == 0:
            self.remove_previous_save_local_path(local_path)
