"""v1 PPO trainer: rollout and training are decoupled through a replay buffer.

The producer side turns dataset prompts into ``n`` agent-loop sessions each, whose trajectories land in the
replay buffer keyed ``{uid}_{session}_{index}``; the consumer side samples complete groups, runs the same
learning phase as the synchronous trainer (reward -> log-probs -> advantages -> updates) and decides, through
hooks, when weights reach the rollout engines. Three modes subclass this file's ``PPOTrainer``: ``sync``,
``colocate_async`` and ``separate_async``.

Everything runs in the trainer's process: rollout requests are coroutines on one event loop and the in-process
engine advances whenever the loop is idle, so "asynchronous" here means *requests stay in flight across
training steps* (partial rollout), not concurrent use of one GPU by two programs.

Parity target: ``verl/trainer/ppo/v1/trainer_base.py`` (class :118, ``_build_replay_buffer`` :142, ``fit`` :387-507,
``step`` :509, ``_step_once`` :538-588, hooks :592-637, registry :1888-1906) and ``agent_loop_tq.py:53-257``.
"""

from __future__ import annotations

import asyncio
import os
import time
import uuid
from typing import Any, Optional

import numpy as np
import torch

from ....experimental.agent_loop.agent_loop import AgentLoopWorker
from ....protocol import DataProto
from ....utils.profiler import marked_timer
from ....utils.tracking import Tracking
from ....workers.rollout.llm_server import LLMServerManager
from ..ray_trainer import RayPPOTrainer, compute_response_mask
from .replay_buffer import ReplayBuffer

__all__ = ["PPOTrainer", "register_trainer", "get_trainer_cls", "AgentLoopWorkerTQ"]

_TRAINERS: dict[str, type] = {}


def register_trainer(mode: str):
    def deco(cls):
        _TRAINERS[mode] = cls
        cls.trainer_mode = mode
        return cls

    return deco


def get_trainer_cls(mode: str) -> type:
    from . import trainer_colocate_async, trainer_separate_async, trainer_sync  # noqa: F401  (self-registering)

    if mode not in _TRAINERS and mode in ("separation", "one_step_off"):
        from ....experimental.one_step_off_policy import ray_trainer  # noqa: F401
    if mode not in _TRAINERS:
        raise ValueError(f"unknown trainer mode '{mode}' (known: {sorted(_TRAINERS)})")
    return _TRAINERS[mode]


class AgentLoopWorkerTQ(AgentLoopWorker):
    """Agent-loop worker that writes each finished session into the replay buffer instead of returning a batch."""

    def __init__(self, *args, replay_buffer: ReplayBuffer, version_fn, **kwargs):
        super().__init__(*args, **kwargs)
        self.rb, self.version_fn = replay_buffer, version_fn

    async def run_session(self, uid: str, session: int, agent_name: str, sampling_params: dict, kwargs: dict,
                          partition_id: str = "train") -> None:
        try:
            got = await self._run_one(agent_name, sampling_params, kwargs)
            # a session may hand back several training rows (index 0, 1, ...); the last one closes the session and carries
            # its outcome; a session that returns nothing usable counts as failed
            outs = [o for o in (got if isinstance(got, (list, tuple)) else [got]) if o is not None]
            if not outs:
                raise RuntimeError("the agent loop returned no trajectory")
            for j, out in enumerate(outs):
                fields = {"prompt_ids": out.prompt_ids, "response_ids": out.response_ids, "response_mask": out.response_mask,
                          "response_logprobs": out.response_logprobs, "reward_score": out.reward_score, "num_turns": out.num_turns,
                          "reward_extra_info": dict(out.extra_fields.get("reward_extra_info", {}) or {}), "output": out}
                self.rb.add_trajectory(uid, session, j, fields, self.version_fn(), failed=False, last=j == len(outs) - 1,
                                       partition_id=partition_id)
        except asyncio.CancelledError:
            raise
        except Exception as e:  # a failed session still completes its group
            self.rb.add_trajectory(uid, session, 0, {"error": repr(e)}, self.version_fn(), failed=True, partition_id=partition_id)


class PPOTrainer(RayPPOTrainer):
    trainer_mode = "base"
    fully_async_client = False

    # ------------------------------------------------------------------ set-up
    def init(self) -> None:
        self.init_workers()
        self._loop = asyncio.new_event_loop()
        self._setup_rollout()
        self.replay_buffer = self._build_replay_buffer()
        self.worker_tq = AgentLoopWorkerTQ(self.config, self.server_manager.client(), self.tokenizer, None,
                                           replay_buffer=self.replay_buffer, version_fn=lambda: self.param_version,
                                           teacher_server_manager=getattr(self, "teacher_server_manager", None))
        self.param_version = 0
        self._tasks: set = set()
        self._prompt_iter = None
        self._epoch = 0
        self.on_init_end()

    def _local_engines(self) -> list:
        wg = self.actor_rollout_wg
        workers = getattr(wg, "_workers", [])
        engines = [getattr(w, "rollout", None) for w in workers]
        if not engines or any(e is None or not hasattr(e, "step") for e in engines):
            raise RuntimeError("the v1 trainers drive in-process rollout engines: use trainer.worker_group=inprocess or spmd")
        return engines

    def _setup_rollout(self) -> None:
        rc = self.config.actor_rollout_ref.rollout
        engines = self._local_engines()
        self.server_manager = self._loop.run_until_complete(
            LLMServerManager.create(rc, model_config=None, engines=engines, fully_async=self.fully_async_client))

    def _tc(self, key: str, default=None):
        t = self.config.trainer
        v1 = t.get("v1") if hasattr(t, "get") else None
        if v1 is not None and v1.get(key) is not None:
            return v1.get(key)
        return t.get(key, default)

    def _build_replay_buffer(self) -> ReplayBuffer:
        algo = self.config.algorithm
        fg = algo.get("filter_groups") or {}
        metric = fg.get("metric") if fg and fg.get("enable", False) else None
        return ReplayBuffer(self.trainer_mode, n=int(self.config.actor_rollout_ref.rollout.n),
                            max_off_policy_threshold=int(self._tc("max_off_policy_threshold", 1)),
                            max_off_policy_strategy=str(self._tc("max_off_policy_strategy", "drop")),
                            filter_groups_metric=metric, refill_fn=self._refill,
                            sync_refill_failed_groups=bool(self._tc("sync_refill_failed_groups", False)))

    # ------------------------------------------------------------------ producer
    def _next_prompts(self, k: int) -> list[dict]:
        """k single-prompt dictionaries from the dataloader (cycling epochs)."""
        out: list[dict] = []
        while len(out) < k:
            if self._prompt_iter is None:
                self._prompt_iter = iter(self.train_dataloader)
            try:
                bd = next(self._prompt_iter)
            except StopIteration:
                self._prompt_iter = None
                self._epoch += 1
                if self._epoch >= self.config.trainer.total_epochs and not out:
                    break
                continue
            b = len(next(iter(bd.values())))
            for i in range(b):
                out.append({k2: (v[i] if not isinstance(v, torch.Tensor) else v[i]) for k2, v in bd.items()})
        return out[:k] if len(out) > k else out

    def _refill(self, k: int) -> None:
        self._submit_prompts(self._next_prompts(k))

    def _submit_prompts(self, prompts: list[dict], partition_id: str = "train") -> int:
        rc = self.config.actor_rollout_ref.rollout
        sp = dict(temperature=float(rc.temperature), top_p=float(rc.get("top_p", 1.0)), top_k=int(rc.get("top_k", -1)),
                  logprobs=True)
        default_loop = self.worker_tq.default_loop
        for p in prompts:
            uid = str(p.get("uid") or uuid.uuid4().hex)
            kw = {k: v for k, v in p.items() if not isinstance(v, torch.Tensor)}
            if "raw_prompt" not in kw and "input_ids" in p:
                ids, am = p["input_ids"], p.get("attention_mask")
                kw["raw_prompt_ids"] = (ids[am.bool()] if am is not None else ids).tolist()
            self.replay_buffer.add_prompt(uid, kw, self.param_version, partition_id)
            self.replay_buffer.mark_running(uid, partition_id)
            for s in range(int(rc.n)):
                t = self._loop.create_task(self.worker_tq.run_session(uid, s, str(kw.get("agent_name", default_loop)), sp, kw, partition_id))
                self._tasks.add(t)
                t.add_done_callback(self._tasks.discard)
        return len(prompts)

    def _pump(self, seconds: float = 0.0) -> None:
        """Let the event loop (and with it the in-process engines) make progress."""
        self._loop.run_until_complete(asyncio.sleep(seconds))

    # ------------------------------------------------------------------ consumer
    def _batch_from_meta(self, meta) -> DataProto:
        recs = self.replay_buffer.q.get_data(meta)
        outs, uids, keys = [], [], []
        for key, r in zip(meta.keys, recs):
            if "output" in r:
                outs.append(r["output"])
                uids.append(key.rsplit("_", 2)[0])
                keys.append(key)
        shell = DataProto.from_dict(tensors={"dummy": torch.zeros(len(outs), 1)}, meta_info={})
        batch = self.worker_tq._postprocess(outs, shell)
        batch.meta_info.pop("timing", None)
        batch.meta_info.pop("reward_extra_keys", None)
        batch.non_tensor_batch["uid"] = np.array(uids, dtype=object)
        batch.non_tensor_batch["__traj_key__"] = np.array(keys, dtype=object)
        prompts = {u: self.replay_buffer.q.get([u], None, meta.partition_id)[0].get("prompt", {}) for u in set(uids)}
        for k in sorted({k for p in prompts.values() for k in p}):
            if k in batch.non_tensor_batch or k in ("uid",):
                continue
            arr = np.empty(len(uids), dtype=object)
            arr[:] = [prompts[u].get(k) for u in uids]
            batch.non_tensor_batch[k] = arr
        if "response_mask" not in batch.batch.keys():
            batch.batch["response_mask"] = compute_response_mask(batch)
        batch.meta_info["temperature"] = self.config.actor_rollout_ref.rollout.temperature
        return self._to_device(batch)

    def _compute_advantage(self, batch: DataProto, **kw) -> DataProto:
        keys = batch.non_tensor_batch.get("__traj_key__")
        if keys is not None:
            from .utils import compute_advantage_for_multi_trajectories, has_multi_trajectory_sessions

            if has_multi_trajectory_sessions(keys.tolist()):
                return compute_advantage_for_multi_trajectories(batch, keys.tolist(), **kw)
        return super()._compute_advantage(batch, **kw)

    def _step_once(self, metrics: dict, timing_raw: dict) -> Optional[DataProto]:
        # train_batch_size counts prompts of the whole job; a controller-replicated rank trains on its share
        _, dp_world = self._dp_rank_world()
        bs = max(1, int(self.config.data.train_batch_size) // max(1, dp_world))
        self.on_sample_begin()
        with marked_timer("gen", timing_raw, color="red"):
            meta = self.replay_buffer.sample(bs, current_version=self.param_version, pump=self._pump)
        if meta is None:
            return None
        self.on_sample_end()
        batch = self._batch_from_meta(meta)
        batch = self.learn_phase(batch, metrics, timing_raw)
        self.replay_buffer.release(meta)
        metrics.update(self.replay_buffer.pop_metrics())
        return batch

    def step(self) -> Optional[tuple[dict, dict]]:
        """One trainer step = ``parameter_sync_step`` optimizer rounds, then the weight hand-over hook."""
        metrics: dict[str, Any] = {}
        timing_raw: dict[str, float] = {}
        batch = None
        with marked_timer("step", timing_raw):
            self.on_step_begin()
            rounds = max(1, int(self._tc("parameter_sync_step", 1)))
            if rounds == 1:
                batch = self._step_once(metrics, timing_raw)
                if batch is None:
                    return None
            else:
                # several optimizer rounds per weight hand-over: the step's record reduces the rounds' records by name
                from .utils import StepMetricsAggregator

                agg = StepMetricsAggregator()
                for _ in range(rounds):
                    m: dict[str, Any] = {}
                    batch = self._step_once(m, timing_raw)
                    if batch is None:
                        return None
                    agg.add_step_metrics(m, len(batch))
                metrics.update(agg.get_aggregated_metrics())
            self.on_step_end(batch, metrics, timing_raw)
        return self.finish_step(batch, metrics, timing_raw)

    def fit(self) -> None:
        cfg = self.config
        rank, _ = self._dp_rank_world()
        logger = Tracking(project_name=cfg.trainer.get("project_name", "verl_b200"), experiment_name=cfg.trainer.get("experiment_name", "run"),
                          default_backend=cfg.trainer.get("logger", ["console"]) if rank == 0 else [], config=cfg)
        if not hasattr(self, "replay_buffer"):
            self.init()
        self.global_steps = 0
        self._load_checkpoint()
        self.sync_phase(None, {}, {})
        self.on_train_begin()
        self.global_steps += 1
        while self.global_steps <= self.total_training_steps:
            res = self.step()
            if res is None:
                break
            metrics, timing_raw = res
            sf = cfg.trainer.get("save_freq", -1)
            if sf and sf > 0 and (self.global_steps % sf == 0 or self.global_steps == self.total_training_steps):
                self._save_checkpoint()
            metrics["training/global_step"] = self.global_steps
            metrics["training/param_version"] = self.param_version
            logger.log(data=metrics, step=self.global_steps)
            self.global_steps += 1
        self.shutdown()

    # ------------------------------------------------------------------ checkpoint of the buffer
    def _save_checkpoint(self) -> None:
        """Actor / critic / dataloader as in the synchronous trainer; the asynchronous modes also keep the replay buffer:
        groups that are finished but not yet trained on, and the prompts whose trajectories are still being generated.
        Parity target: ``verl/trainer/ppo/v1/trainer_base.py:887-960``."""
        super()._save_checkpoint()
        if self.replay_buffer.is_async:
            rank, _ = self._dp_rank_world()
            root = os.path.join(self.config.trainer.default_local_dir, f"global_step_{self.global_steps}")
            self.replay_buffer.q.save_checkpoint(os.path.join(root, "transfer_queue" if rank == 0 else f"transfer_queue_rank{rank}"),
                                                 metadata={"global_steps": self.global_steps, "param_version": self.param_version})

    def _load_checkpoint(self) -> int:
        step = super()._load_checkpoint()
        if step and self.replay_buffer.is_async:
            rank, _ = self._dp_rank_world()
            folder = os.path.join(self.config.trainer.default_local_dir, f"global_step_{step}") \
                if self.config.trainer.get("resume_mode", "auto") != "resume_path" else str(self.config.trainer.get("resume_from_path"))
            path = os.path.join(folder, "transfer_queue" if rank == 0 else f"transfer_queue_rank{rank}")
            if os.path.exists(os.path.join(path, "state.pt")):
                meta = self.replay_buffer.q.load_checkpoint(path)
                self.param_version = int(meta.get("param_version", self.param_version))
                self._reissue_inflight_prompts()
        return step

    def _reissue_inflight_prompts(self, partition_id: str = "train") -> int:
        """Prompt groups that were pending or running when the checkpoint was written start again from their stored prompt:
        the partial trajectories they had produced are dropped, their counters reset, their sessions re-submitted under the
        current parameter version. Parity target: ``verl/trainer/ppo/v1/trainer_base.py:849-885``."""
        from .replay_buffer import PENDING, RUNNING

        q = self.replay_buffer.q
        live = q.list_keys(partition_id, lambda k, t: t.get("kind") == "prompt" and t.get("status") in (PENDING, RUNNING))
        if not live:
            return 0
        old = q.list_keys(partition_id, lambda k, t: t.get("kind") == "traj" and t.get("uid") in set(live))
        q.delete(old, partition_id)
        prompts = []
        for uid in live:
            payload = dict(q.get([uid], None, partition_id)[0].get("prompt", {}))
            payload["uid"] = uid
            prompts.append(payload)
            q.delete([uid], partition_id)   # _submit_prompts stores it again with fresh counters
        self._submit_prompts(prompts, partition_id)
        print(f"Re-issued {len(live)} in-flight prompts for step {self.global_steps}; cleared {len(old)} partial trajectories")
        return len(live)

    def shutdown(self) -> None:
        for t in list(self._tasks):
            t.cancel()
        pending = list(self._tasks)

        async def go():
            await asyncio.gather(*pending, return_exceptions=True)

        if pending:
            self._loop.run_until_complete(go())

    # ------------------------------------------------------------------ hooks (modes override)
    def on_init_end(self) -> None: ...

    def on_train_begin(self) -> None: ...

    def on_step_begin(self) -> None: ...

    def on_sample_begin(self) -> None: ...

    def on_sample_end(self) -> None: ...

    def on_step_end(self, batch, metrics: dict, timing_raw: dict) -> None: ...

    # helpers shared by the modes
    def _servers(self) -> list:
        return list(self.server_manager.servers.values())

    def _each_server(self, method: str, *args) -> None:
        async def go():
            await asyncio.gather(*[getattr(s, method)(*args) for s in self._servers()])

        self._loop.run_until_complete(go())

    def _push_weights(self, batch, metrics: dict, timing_raw: dict) -> None:
        self.sync_phase(batch, metrics, timing_raw)
        self.param_version += 1
        self._each_server("set_global_steps", self.param_version)
