"""Consumer side of the fully-asynchronous pipeline and the in-process composition of both sides.

``FullyAsyncTrainer.fit`` repeats: pull ``require_batches x ppo_mini_batch_size`` samples from the message queue
(driving the rollouter while it waits), assemble the batch, run the learning phase, and after every
``trigger_parameter_sync_step`` local updates synchronise weights, which also resets the rollouter's staleness
budget. Rollouter and trainer share one process and one event loop here; with a separate rollout pool the same
classes sit on the two sides of a ``StoreMessageQueue``.

Parity target: ``verl/experimental/fully_async_policy/fully_async_trainer.py`` (``_get_samples_from_queue`` :375,
``fit_step`` :536, ``_fit_update_weights`` :690) and ``fully_async_main.py``.
"""

from __future__ import annotations

import asyncio
import os
import time
from typing import Any, Optional

import numpy as np
import torch

from ...protocol import DataProto
from ...trainer.ppo.ray_trainer import compute_response_mask
from ...trainer.ppo.v1.trainer_base import PPOTrainer
from ...utils.profiler import marked_timer
from ...utils.tracking import Tracking
from .detach_utils import MetricsAggregator, RolloutSample
from .fully_async_rollouter import FullyAsyncRollouter
from .message_queue import MessageQueue
from .param_sync import ParameterSynchronizer

__all__ = ["FullyAsyncTrainer", "assemble_batch_from_rollout_samples"]


def assemble_batch_from_rollout_samples(samples: list[RolloutSample], postprocess, to_device) -> DataProto:
    outs, uids, v0, v1 = [], [], [], []
    for s in samples:
        for o in s.trajectories:
            outs.append(o)
            uids.append(s.uid)
            v0.append(s.param_version_start)
            v1.append(s.param_version_end)
    shell = DataProto.from_dict(tensors={"dummy": torch.zeros(len(outs), 1)}, meta_info={})
    batch = postprocess(outs, shell)
    batch.meta_info.pop("timing", None)
    batch.meta_info.pop("reward_extra_keys", None)
    batch.non_tensor_batch["uid"] = np.array(uids, dtype=object)
    batch.non_tensor_batch["param_version_start"] = np.array(v0, dtype=np.int64)
    batch.non_tensor_batch["param_version_end"] = np.array(v1, dtype=np.int64)
    keys = sorted({k for s in samples for k in s.prompt if k not in ("uid", "raw_prompt_ids")})
    for k in keys:
        arr = np.empty(len(uids), dtype=object)
        arr[:] = [s.prompt.get(k) for s in samples for _ in s.trajectories]
        batch.non_tensor_batch.setdefault(k, arr)
    if "response_mask" not in batch.batch.keys():
        batch.batch["response_mask"] = compute_response_mask(batch)
    return to_device(batch)


class FullyAsyncTrainer(PPOTrainer):
    trainer_mode = "fully_async"
    fully_async_client = True

    def _ac(self, key: str, default=None):
        ac = self.config.get("async_training") if hasattr(self.config, "get") else None
        return default if ac is None or ac.get(key) is None else ac.get(key)

    def on_init_end(self) -> None:
        rc = self.config.actor_rollout_ref.rollout
        mini = int(self.config.actor_rollout_ref.actor.ppo_mini_batch_size)
        self.required_samples = int(self._ac("require_batches", 1)) * mini
        self.trigger = int(self._ac("trigger_parameter_sync_step", 1))
        self.mq = MessageQueue(max_queue_size=int(self._ac("max_queue_size", 16 * self.required_samples)))
        sp = dict(temperature=float(rc.temperature), top_p=float(rc.get("top_p", 1.0)), top_k=int(rc.get("top_k", -1)), logprobs=True)
        total = self._ac("total_rollout_samples")

        def prompt_source(k: int) -> list[dict]:
            out = []
            for p in self._next_prompts(k):
                kw = {a: b for a, b in p.items() if not isinstance(b, torch.Tensor)}
                if "raw_prompt" not in kw and "input_ids" in p:
                    ids, am = p["input_ids"], p.get("attention_mask")
                    kw["raw_prompt_ids"] = (ids[am.bool()] if am is not None else ids).tolist()
                out.append(kw)
            return out

        self.rollouter = FullyAsyncRollouter(self.worker_tq, self.server_manager, self.mq, prompt_source, n=int(rc.n),
                                             sampling_params=sp, required_samples=self.required_samples,
                                             trigger_parameter_sync_step=self.trigger,
                                             staleness_threshold=float(self._ac("staleness_threshold", 1.0)),
                                             max_concurrent_samples=self._ac("max_concurrent_samples"), total_samples=total)
        self.synchronizer = ParameterSynchronizer(
            pause_fn=lambda: (self._each_server("abort_all_requests"), self._pump()),
            resume_fn=lambda: self._each_server("resume_generation"),
            transfer_fn=lambda v: self.actor_rollout_wg.update_weights(v),
            message_queue=self.mq,
            set_version_fn=lambda v: (setattr(self, "_rollouter_step_timing", self.rollouter.update_param_version(v)),
                                      self._each_server("set_global_steps", v)))
        self._rollouter_step_timing: dict = {}
        # one pool: every GPU of the job switches between generation and training ("hybrid" in the utilisation formula)
        n_gpus = int(self.config.trainer.get("n_gpus_per_node", 1) or 1) * int(self.config.trainer.get("nnodes", 1) or 1)
        self.aggregator = MetricsAggregator(total_gpus=n_gpus, hybrid_gpus=n_gpus, standalone_gpus=0)
        self.local_updates = 0

    def _drive(self) -> None:
        async def go():
            self.rollouter.feed()
            await asyncio.sleep(0)

        self._loop.run_until_complete(go())

    def _get_samples_from_queue(self, timing_raw: dict) -> Optional[list[RolloutSample]]:
        got: list[RolloutSample] = []
        idle0 = time.time()
        while len(got) < self.required_samples:
            item = self.mq.get_sample(timeout=0.0)
            if item is not None:
                got.append(item[0])
                continue
            self._drive()
            if not self.rollouter.running and self.mq.get_queue_size() == 0 and self.rollouter._should_pause_generation():
                if self.rollouter.total_samples is not None and self.rollouter.submitted >= self.rollouter.total_samples:
                    return None  # the stream ended
                # paused on staleness with nothing in flight: only a weight sync can make progress
                break
        timing_raw["wait_samples"] = time.time() - idle0
        return got or None

    def fit_step(self) -> Optional[tuple[dict, dict]]:
        metrics: dict[str, Any] = {}
        timing_raw: dict[str, float] = {}
        self._bind_step(metrics, timing_raw)
        with marked_timer("step", timing_raw):
            self._each_server("resume_generation")
            with marked_timer("gen", timing_raw, color="red"):
                samples = self._get_samples_from_queue(timing_raw)
            if not samples:
                return None
            self._each_server("abort_all_requests")  # the GPU is time-shared: generation rests while we train
            self._pump()
            batch = assemble_batch_from_rollout_samples(samples, self.worker_tq._postprocess, self._to_device)
            batch.meta_info["temperature"] = self.config.actor_rollout_ref.rollout.temperature
            spans = [s.staleness_span for s in samples]
            age = [self.param_version - s.param_version_start for s in samples]
            metrics.update({"fully_async/staleness_span/mean": float(np.mean(spans)), "fully_async/staleness_span/max": float(np.max(spans)),
                            "fully_async/sample_age/mean": float(np.mean(age)), "fully_async/sample_age/max": float(np.max(age)),
                            "fully_async/queue_size": float(self.mq.get_queue_size())})
            t_alloc = time.time()
            batch = self.learn_phase(batch, metrics, timing_raw)
            self.local_updates += 1
            if self.local_updates % self.trigger == 0:
                self._fit_update_weights()
            self._record_train_resource_utilization(time.time() - t_alloc)
        # generation rests while this pool trains, so the time the trainer waited for samples IS the pool's generation turn
        timing_raw["wait_for_enough_samples"] = timing_raw.get("gen", 0.0)
        metrics.update(self.rollouter.statistics())
        return self.finish_step(batch, metrics, timing_raw)

    # phases of ``learn_phase`` that are training compute (the rest of a step's allocated time is hand-over and waiting)
    _TRAIN_COMPUTE_TIMING_KEYS = ("reward", "old_log_prob", "ref", "values", "adv", "update_critic", "update_actor")

    def _record_train_resource_utilization(self, allocated_time: float) -> None:
        """Raw seconds, not a ratio: the aggregator sums both over the steps of a synchronisation cycle and divides once
        (``dynamic_resource/train_resource_utilization``). Numerator: the training-compute phases; denominator: the wall
        clock from the first of them to the end of the weight hand-over."""
        self.metrics["dynamic_resource/train_compute_time_s"] = sum(self.timing_raw.get(k, 0.0) for k in self._TRAIN_COMPUTE_TIMING_KEYS)
        self.metrics["dynamic_resource/train_allocated_time_s"] = float(allocated_time)

    def _fit_update_weights(self) -> None:
        """Push the weights to the rollouter through the parameter synchroniser and open a new parameter version (the
        base class's in-place hand-over is what ``fit`` uses once, before the first step)."""
        metrics, timing_raw = self.metrics, self.timing_raw
        with marked_timer("update_weights", timing_raw, color="red"):
            self.param_version += 1
            res = self.synchronizer.sync_weights(self.param_version)
        res = res if isinstance(res, dict) else {}
        metrics["timing_s/param_sync"] = float(res.get("timing_s/param_sync", 0.0))
        metrics["fully_async/param_version"] = self.param_version
        metrics.update(self._rollouter_step_timing or {})   # the producer's record of the step that this sync closed

    def step(self):
        return self.fit_step()

    # ------------------------------------------------------------------ checkpoint
    def _ckpt_folder(self, step: int) -> str:
        t = self.config.trainer
        if t.get("resume_mode", "auto") == "resume_path" and t.get("resume_from_path") and f"global_step_{step}" in str(t.get("resume_from_path")):
            return str(t.get("resume_from_path"))
        return os.path.join(str(t.default_local_dir), f"global_step_{step}")

    def _save_checkpoint(self) -> None:
        """Actor / dataloader as in the synchronous trainer, plus the producer's side: counters, samples still queued for the
        trainer and the prompts that were in flight (``FullyAsyncRollouter.state_dict``)."""
        super()._save_checkpoint()
        self.rollouter.save_checkpoint(self._ckpt_folder(self.global_steps))
        torch.save({"local_updates": self.local_updates, "param_version": self.param_version},
                   os.path.join(self._ckpt_folder(self.global_steps), "fully_async_trainer.pt"))

    def _load_checkpoint(self) -> int:
        step = super()._load_checkpoint()
        if step and hasattr(self, "rollouter"):
            folder = self._ckpt_folder(step)
            if self.rollouter.load_checkpoint(folder):
                own = os.path.join(folder, "fully_async_trainer.pt")
                if os.path.exists(own):
                    st = torch.load(own, map_location="cpu", weights_only=False)
                    self.local_updates, self.param_version = int(st["local_updates"]), int(st["param_version"])
                self.rollouter.param_version = self.param_version
                print(f"Resumed the rollouter: {self.mq.get_queue_size()} queued samples, {len(self.rollouter._replay)} prompts re-issued")
        return step

    def fit(self) -> None:
        cfg = self.config
        logger = Tracking(project_name=cfg.trainer.get("project_name", "verl_b200"), experiment_name=cfg.trainer.get("experiment_name", "run"),
                          default_backend=cfg.trainer.get("logger", ["console"]), config=cfg)
        if not hasattr(self, "replay_buffer"):
            self.init()
        self.global_steps = 0
        resumed = int(self._load_checkpoint() or 0)
        self._bind_step({}, {})
        super()._fit_update_weights()
        self._each_server("wake_up")
        if self.val_reward_fn is not None and cfg.trainer.get("val_before_train", False):
            val = self._validate()
            if val:
                logger.log(data=val, step=self.global_steps)
            if cfg.trainer.get("val_only", False):
                return
        self.global_steps = resumed + 1
        while self.global_steps <= self.total_training_steps:
            res = self.fit_step()
            if res is None:
                break
            metrics, timing_raw = res
            self.aggregator.add_step_metrics(metrics, self.required_samples)
            if self.local_updates % self.trigger == 0:
                agg = self.aggregator.get_aggregated_metrics(
                    rollout_resource_utilization=(self._rollouter_step_timing or {}).get("dynamic_resource/rollout_resource_utilization"))
                agg["training/global_step"] = self.global_steps
                self.last_aggregated_metrics = agg
                self.is_last_step = self.global_steps >= self.total_training_steps
                self._bind_step(agg, timing_raw)
                self._fit_validate()          # test_freq counts training steps; runs between two cycles, generation resting
                self._fit_save_checkpoint()
                logger.log(data=agg, step=self.global_steps)
                self.aggregator.reset()
            self.global_steps += 1
        for t in list(self.rollouter.running.values()):
            t.cancel()
        self.shutdown()
