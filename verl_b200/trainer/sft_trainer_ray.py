"""SFT driven by a single controller: the driver owns data loading and logging and calls ``train_batch`` /
``infer_batch`` on a worker group (one ``TrainingWorker`` per GPU), which shards each global batch over the
data-parallel ranks. ``trainer.worker_group`` picks the back-end (multiprocess, inprocess, ray).

Parity target: ``verl/trainer/sft_trainer_ray.py``. The SPMD variant (``torchrun``) is ``sft_trainer.py``.
"""

from __future__ import annotations

import os
import sys
import time
from functools import partial
from typing import Optional, Sequence

import torch

from ..protocol import DataProto
from ..single_controller.base import ClassWithInitArgs
from ..utils.checkpoint.checkpoint_manager import find_latest_ckpt_path, rotate_checkpoints
from ..utils.config import load_config, omega_conf_to_dataclass
from ..utils.dataset.multiturn_sft_dataset import MultiTurnSFTDataset, SyntheticSFTDataset, sft_collate
from ..utils.dataset.stateful import StatefulDataLoader
from ..utils.tracking import Tracking
from ..workers.config import CheckpointConfig, FSDPEngineConfig, HFModelConfig, OptimizerConfig, TrainingWorkerConfig
from ..workers.engine_workers import TrainingWorker
from ..workers.utils.losses import sft_loss

CONFIG_DIR = os.path.join(os.path.dirname(__file__), "config")

__all__ = ["SFTTrainerRay", "SFTWorker", "main"]


class SFTWorker(TrainingWorker):
    """TrainingWorker that builds itself from the plain SFT config (so that the init args pickle to any back-end)."""

    def __init__(self, config, total_steps: int):
        mc = omega_conf_to_dataclass(config.model, HFModelConfig)
        ec = omega_conf_to_dataclass(config.engine, FSDPEngineConfig)
        for k in ("micro_batch_size_per_gpu", "max_token_len_per_gpu", "use_dynamic_bsz"):
            if config.data.get(k) is not None:
                object.__setattr__(ec, k, config.data.get(k))
        oc = omega_conf_to_dataclass(config.optim, OptimizerConfig)
        oc.total_training_steps = total_steps
        super().__init__(TrainingWorkerConfig(model_type="language_model", model_config=mc, engine_config=ec, optimizer_config=oc,
                                              checkpoint_config=omega_conf_to_dataclass(config.checkpoint, CheckpointConfig)))
        self.reset()
        self.set_loss_fn(partial(sft_loss, None))


class SFTTrainerRay:
    def __init__(self, config, worker_group_cls=None, worker_group_kwargs: Optional[dict] = None):
        self.config = config
        mc = omega_conf_to_dataclass(config.model, HFModelConfig)
        d = config.data
        if d.get("train_files"):
            tok = mc.get_tokenizer()
            self.train_ds = MultiTurnSFTDataset(d.train_files, tok, d)
            self.val_ds = MultiTurnSFTDataset(d.val_files, tok, d) if d.get("val_files") else None
        else:
            syn = d.get("synthetic") or {}
            n = int(syn.get("num_samples", int(d.train_batch_size) * 4))
            self.train_ds = SyntheticSFTDataset(n, int(d.max_length), mc.arch.vocab_size, seed=int(syn.get("seed", 0)))
            self.val_ds = SyntheticSFTDataset(max(8, n // 8), int(d.max_length), mc.arch.vocab_size, seed=7919)
        coll = partial(sft_collate, pad_token_id=mc.arch.pad_token_id or 0)
        self.train_loader = StatefulDataLoader(self.train_ds, batch_size=int(d.train_batch_size), collate_fn=coll, drop_last=True,
                                               shuffle=True, seed=int(config.trainer.get("seed", 1)))
        self.val_loader = StatefulDataLoader(self.val_ds, batch_size=int(d.train_batch_size), collate_fn=coll, drop_last=True) if self.val_ds else None
        steps = len(self.train_loader) * int(config.trainer.total_epochs)
        self.total_steps = int(config.trainer.get("total_training_steps") or steps)
        if worker_group_cls is None:
            from ..single_controller.local import InProcessWorkerGroup, MultiprocessWorkerGroup

            n_gpus = int(config.trainer.get("n_gpus_per_node", 1)) * int(config.trainer.get("nnodes", 1))
            kind = config.trainer.get("worker_group", "auto")
            if kind == "ray":
                from ..single_controller.ray import RayWorkerGroup as worker_group_cls
            else:
                worker_group_cls = InProcessWorkerGroup if (n_gpus == 1 or kind == "inprocess") else MultiprocessWorkerGroup
            self.n_workers = n_gpus
        else:
            self.n_workers = int(config.trainer.get("n_gpus_per_node", 1)) * int(config.trainer.get("nnodes", 1))
        self.wg = worker_group_cls(self.n_workers, ClassWithInitArgs(SFTWorker, config=config, total_steps=self.total_steps),
                                   **(worker_group_kwargs or {}))
        self.global_step = 0

    def _proto(self, batch: dict) -> DataProto:
        return DataProto.from_dict(tensors=dict(batch))

    def validate(self) -> Optional[float]:
        if self.val_loader is None:
            return None
        num = den = 0.0
        for batch in self.val_loader:
            out = self.wg.infer_batch(self._proto(batch))
            lp, m = out.batch["log_probs"].cpu(), batch["response_mask"].float()
            num += float(-(lp * m).sum())
            den += float(m.sum())
        return num / max(den, 1.0) if den else None

    def save(self) -> None:
        t = self.config.trainer
        path = os.path.join(t.default_local_dir, f"global_step_{self.global_step}")
        self.wg.save_checkpoint(path, None, self.global_step, t.get("max_ckpt_to_keep"))
        torch.save(self.train_loader.state_dict(), os.path.join(path, "data.pt"))
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
        self.wg.load_checkpoint(path)
        self.global_step = int(str(path).split("global_step_")[-1])
        dp = os.path.join(path, "data.pt")
        if os.path.exists(dp):
            self.train_loader.load_state_dict(torch.load(dp, weights_only=False))

    def fit(self) -> dict:
        t = self.config.trainer
        logger = Tracking(t.project_name, t.experiment_name, t.get("logger", ["console"]), self.config)
        self.resume()
        last: dict = {}
        for _ in range(int(t.total_epochs)):
            for batch in self.train_loader:
                if self.global_step >= self.total_steps:
                    return last
                t0 = time.time()
                out = self.wg.train_batch(self._proto(batch))
                m = out.meta_info.get("metrics", {}) if isinstance(out, DataProto) else {}
                from .ppo.metric_utils import reduce_metrics

                m = reduce_metrics(m)
                self.global_step += 1
                last = {"train/loss": m.get("loss", 0.0), "train/grad_norm": m.get("grad_norm", 0.0), "train/lr": m.get("lr", 0.0),
                        "train/tokens_per_s": float(batch["attention_mask"].sum()) / max(time.time() - t0, 1e-9)}
                tf, sf = t.get("test_freq", -1), t.get("save_freq", -1)
                if tf and tf > 0 and self.global_step % tf == 0:
                    v = self.validate()
                    if v is not None:
                        last["val/loss"] = v
                logger.log(last, step=self.global_step)
                if sf and sf > 0 and self.global_step % sf == 0:
                    self.save()
        return last


def main(argv: Optional[Sequence[str]] = None):
    argv = list(sys.argv[1:] if argv is None else argv)
    trainer = SFTTrainerRay(load_config(CONFIG_DIR, "sft_trainer_engine", argv))
    return trainer.fit()


if __name__ == "__main__":
    main()
