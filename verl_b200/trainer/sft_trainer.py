"""Supervised fine-tuning, SPMD: ``torchrun -m verl_b200.trainer.sft_trainer key=value ...``.

Every rank builds a :class:`TrainingWorker` in-process with the SFT loss, reads its shard of the data, and steps
through the native sharded engine. Parity target: ``verl/trainer/sft_trainer.py`` (``SFTTrainer`` :159-449,
``run_sft`` :452, entry :461).
"""

from __future__ import annotations

import os
import sys
import time
from functools import partial
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..protocol import DataProto
from ..utils.checkpoint.checkpoint_manager import find_latest_ckpt_path, rotate_checkpoints
from ..utils.config import load_config, omega_conf_to_dataclass
from ..utils.dataset.multiturn_sft_dataset import MultiTurnSFTDataset, SyntheticSFTDataset, sft_collate
from ..utils.dataset.stateful import ShardedRandomSampler, StatefulDataLoader
from ..utils.device import get_device_name
from ..utils.distributed import initialize_global_process_group
from ..utils.tracking import Tracking
from ..workers.config import CheckpointConfig, FSDPEngineConfig, HFModelConfig, OptimizerConfig, TrainingWorkerConfig
from ..workers.engine_workers import TrainingWorker
from ..workers.utils.losses import sft_loss
from .config import CONFIG_DIR

__all__ = ["SFTTrainer", "run_sft", "main"]


class SFTTrainer:
    def __init__(self, config):
        self.config = config
        _, self.rank, self.world = initialize_global_process_group()
        self.device = torch.device("cuda", torch.cuda.current_device()) if get_device_name() == "cuda" else torch.device("cpu")
        mc = omega_conf_to_dataclass(config.model, HFModelConfig)
        ec = omega_conf_to_dataclass(config.engine, FSDPEngineConfig)
        for src, dst in (("micro_batch_size_per_gpu", "micro_batch_size_per_gpu"), ("max_token_len_per_gpu", "max_token_len_per_gpu"),
                         ("use_dynamic_bsz", "use_dynamic_bsz")):
            if config.data.get(src) is not None:
                object.__setattr__(ec, dst, config.data.get(src))
        oc = omega_conf_to_dataclass(config.optim, OptimizerConfig)
        self.model_config = mc
        self._build_data()
        steps = len(self.train_loader) * int(config.trainer.total_epochs)
        if config.trainer.get("total_training_steps"):
            steps = int(config.trainer.total_training_steps)
        self.total_steps = steps
        oc.total_training_steps = steps
        self.worker = TrainingWorker(TrainingWorkerConfig(model_type="language_model", model_config=mc, engine_config=ec,
                                                          optimizer_config=oc,
                                                          checkpoint_config=omega_conf_to_dataclass(config.checkpoint, CheckpointConfig)))
        self.worker.reset()
        self.worker.set_loss_fn(partial(sft_loss, None))
        self.global_step = 0

    def _build_data(self) -> None:
        d = self.config.data
        tok = self.model_config.get_tokenizer()
        if d.get("train_files"):
            self.train_ds = MultiTurnSFTDataset(d.train_files, tok, d)
            self.val_ds = MultiTurnSFTDataset(d.val_files, tok, d) if d.get("val_files") else None
        else:
            syn = d.get("synthetic") or {}
            n = int(syn.get("num_samples", int(d.train_batch_size) * 4))
            V = self.model_config.arch.vocab_size
            self.train_ds = SyntheticSFTDataset(n, int(d.max_length), V, seed=int(syn.get("seed", 0)))
            self.val_ds = SyntheticSFTDataset(max(8, n // 8), int(d.max_length), V, seed=7919)
        per_rank = int(d.train_batch_size) // self.world
        assert per_rank >= 1, "train_batch_size must be >= world size"
        pad = self.model_config.arch.pad_token_id or 0
        coll = partial(sft_collate, pad_token_id=pad)
        self.train_loader = StatefulDataLoader(self.train_ds, batch_size=per_rank, collate_fn=coll, drop_last=True,
                                               sampler=ShardedRandomSampler(len(self.train_ds), int(self.config.trainer.get("seed", 1)),
                                                                            self.rank, self.world))
        self.val_loader = None
        if self.val_ds is not None:
            self.val_loader = StatefulDataLoader(self.val_ds, batch_size=per_rank, collate_fn=coll, drop_last=True,
                                                 sampler=ShardedRandomSampler(len(self.val_ds), 0, self.rank, self.world))

    def _proto(self, batch: dict) -> DataProto:
        import numpy as np

        non = {}
        for k, v in batch.items():
            if not isinstance(v, torch.Tensor):
                arr = np.empty(len(v), dtype=object)
                arr[:] = list(v)
                non[k] = arr
        return DataProto.from_dict(tensors={k: v.to(self.device) for k, v in batch.items() if isinstance(v, torch.Tensor)},
                                   non_tensors=non)

    def validate(self) -> Optional[float]:
        if self.val_loader is None:
            return None
        losses = []
        for batch in self.val_loader:
            out = self.worker._infer_batch(self._proto(batch))
            lp, m = out.batch["log_probs"], batch["response_mask"].to(self.device).float()
            losses.append((-(lp * m).sum() / m.sum().clamp(min=1)).detach())
        if not losses:
            return None
        loss = torch.stack(losses).mean()
        if self.world > 1:
            from ..utils.distributed import get_data_parallel_group

            dist.all_reduce(loss, group=get_data_parallel_group())
            loss /= self.world
        return float(loss)

    def save(self) -> None:
        t = self.config.trainer
        path = os.path.join(t.default_local_dir, f"global_step_{self.global_step}")
        self.worker.engine.save_checkpoint(path, global_step=self.global_step)
        torch.save(self.train_loader.state_dict(), os.path.join(path, f"data_rank{self.rank}.pt"))
        if self.rank == 0:
            with open(os.path.join(t.default_local_dir, "latest_checkpointed_iteration.txt"), "w") as f:
                f.write(str(self.global_step))
            if t.get("max_ckpt_to_keep"):
                rotate_checkpoints(t.default_local_dir, int(t.max_ckpt_to_keep))

    def resume(self) -> None:
        t = self.config.trainer
        if t.get("resume_mode", "auto") == "disable":
            return
        path = t.get("resume_from_path") if t.get("resume_mode") == "resume_path" else find_latest_ckpt_path(t.default_local_dir)
        if not path:
            return
        self.worker.engine.load_checkpoint(path)
        self.global_step = int(str(path).split("global_step_")[-1])
        dp = os.path.join(path, f"data_rank{self.rank}.pt")
        if os.path.exists(dp):
            self.train_loader.load_state_dict(torch.load(dp, weights_only=False))

    def fit(self) -> dict:
        t = self.config.trainer
        logger = Tracking(t.project_name, t.experiment_name, t.get("logger", ["console"]) if self.rank == 0 else [], self.config)
        self.resume()
        last = {}
        for epoch in range(int(t.total_epochs)):
            for batch in self.train_loader:
                if self.global_step >= self.total_steps:
                    return last
                t0 = time.time()
                m = self.worker._train_batch(self._proto(batch))
                self.global_step += 1
                tokens = float(batch["attention_mask"].sum()) * self.world
                last = {"train/loss": m.get("loss", m.get("sft/loss", 0.0)), "train/grad_norm": m.get("grad_norm", 0.0),
                        "train/lr": m.get("lr", 0.0), "train/tokens_per_s": tokens / max(time.time() - t0, 1e-9),
                        "train/mfu": m.get("perf/mfu", 0.0)}
                tf, sf = t.get("test_freq", -1), t.get("save_freq", -1)
                if tf and tf > 0 and self.global_step % tf == 0:
                    v = self.validate()
                    if v is not None:
                        last["val/loss"] = v
                logger.log(last, step=self.global_step)
                if sf and sf > 0 and self.global_step % sf == 0:
                    self.save()
        return last


def run_sft(config) -> dict:
    trainer = SFTTrainer(config)
    return trainer.fit()


def main(argv: Optional[Sequence[str]] = None):
    argv = list(sys.argv[1:] if argv is None else argv)
    return run_sft(load_config(CONFIG_DIR, "sft_trainer_engine", argv))


if __name__ == "__main__":
    main()
