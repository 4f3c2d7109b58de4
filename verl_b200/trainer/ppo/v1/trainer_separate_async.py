"""``separate_async`` mode: a trainer pool and a standalone rollout pool, plus hybrid switching.

Rank layout under one ``torchrun`` job of ``W`` ranks with ``trainer.v1.rollout_ranks = R``: ranks ``[0, W-R)`` train
(data-parallel among themselves), ranks ``[W-R, W)`` only serve rollout. Prompts travel trainer -> rollout and
trajectory groups travel back through store-backed queues; weights travel from trainer rank 0 to the rollout ranks
every ``parameter_sync_step`` optimizer rounds as an in-place broadcast of the flat parameter buffer.

Trainer ranks are *hybrid*: they also hold a rollout engine that shares the training weights. While a trainer rank
waits for samples it may switch to rollout (pull prompts from the shared queue and generate locally), and switches
back (in-flight requests aborted, partial outputs kept) as soon as a batch is ready. The switch threshold adapts:
switching pays when the expected remaining wait exceeds the measured cost of a round trip.

With ``R = 0`` the mode degenerates to one pool whose weights are handed over every ``parameter_sync_step`` rounds.

Parity target: ``verl/trainer/ppo/v1/trainer_separate_async.py:38-398`` (``HybridEngineMode``,
``switch_to_rollout`` / ``switch_to_trainer``, adaptive threshold, ``add_replicas_to_balancer``).
"""

from __future__ import annotations

import asyncio
import time
import uuid
from enum import Enum
from typing import Optional

import torch
import torch.distributed as dist

from ....experimental.fully_async_policy.message_queue import StoreMessageQueue
from .replay_buffer import FAILURE, FINISHED, ReplayBuffer
from .trainer_base import AgentLoopWorkerTQ, PPOTrainer, register_trainer

__all__ = ["HybridEngineMode", "SwitchController", "SeparateTopology", "RolloutService", "PPOTrainerSeparateAsync"]


class HybridEngineMode(Enum):
    TRAINER = "trainer"
    ROLLOUT = "rollout"


class SwitchController:
    """Decides when an idle trainer rank should lend its GPU to rollout.

    Keeps exponential moving averages of (a) how long the trainer waited for samples per step and (b) what a
    switch round trip costs; switching is worth it once the wait so far exceeds ``ratio`` x cost and the average wait
    says more waiting is likely."""

    def __init__(self, enabled: bool = True, ratio: float = 1.0, ema: float = 0.5, initial_cost_s: float = 0.0):
        self.enabled, self.ratio, self.ema = enabled, ratio, ema
        self.avg_wait_s = 0.0
        self.switch_cost_s = initial_cost_s
        self.num_switches = 0

    def threshold_s(self) -> float:
        return self.ratio * self.switch_cost_s

    def should_switch(self, waited_s: float) -> bool:
        if not self.enabled:
            return False
        expected_remaining = max(self.avg_wait_s - waited_s, 0.0) if self.avg_wait_s > 0 else waited_s
        return waited_s >= self.threshold_s() and (self.avg_wait_s == 0.0 or expected_remaining >= self.threshold_s())

    def record_wait(self, waited_s: float) -> None:
        self.avg_wait_s = waited_s if self.avg_wait_s == 0.0 else self.ema * waited_s + (1 - self.ema) * self.avg_wait_s

    def record_switch_cost(self, cost_s: float) -> None:
        self.num_switches += 1
        self.switch_cost_s = cost_s if self.switch_cost_s == 0.0 else self.ema * cost_s + (1 - self.ema) * self.switch_cost_s


class SeparateTopology:
    """Process groups and queues of the split job; every rank of the job must construct it (collective)."""

    def __init__(self, rollout_ranks: int):
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.R = int(rollout_ranks) if self.world > 1 else 0
        assert 0 <= self.R < self.world, "need at least one trainer rank"
        self.T = self.world - self.R
        self.is_rollout_rank = self.rank >= self.T
        self.trainer_group = self.rollout_group = self.sync_group = None
        self.prompt_q = self.sample_q = None
        if self.R > 0:
            self.trainer_group = dist.new_group(list(range(self.T)))
            self.rollout_group = dist.new_group(list(range(self.T, self.world)))
            self.sync_group = dist.new_group([0] + list(range(self.T, self.world)))
            store = dist.distributed_c10d._get_default_store()
            self.store = dist.PrefixStore("separate_async", store)
            self.prompt_q = StoreMessageQueue(self.store, "prompts")
            self.sample_qs = [StoreMessageQueue(self.store, f"samples/{r}") for r in range(self.T)]

    def version(self, inc: int = 0) -> int:
        return int(self.store.add("weights/version", inc))

    def stop_requested(self, request: bool = False) -> bool:
        return int(self.store.add("stop", 1 if request else 0)) > 0


class _GroupRunner:
    """Shared by rollout ranks and switched trainer ranks: run prompt records through local engines and ship the
    finished groups to the queue of the trainer rank they came from."""

    def __init__(self, worker_tq: AgentLoopWorkerTQ, rb: ReplayBuffer, loop, topo: SeparateTopology, rollout_cfg):
        self.w, self.rb, self.loop, self.topo, self.rc = worker_tq, rb, loop, topo, rollout_cfg
        self.tasks: set = set()
        self.origin: dict[str, int] = {}

    def submit(self, rec: dict, version: int) -> None:
        uid, kw = rec["uid"], rec["kwargs"]
        self.origin[uid] = rec["origin"]
        self.rb.add_prompt(uid, kw, rec.get("start_version", version), "remote")
        self.rb.mark_running(uid, "remote")
        sp = dict(temperature=float(self.rc.temperature), top_p=float(self.rc.get("top_p", 1.0)), top_k=int(self.rc.get("top_k", -1)), logprobs=True)
        for s in range(int(self.rc.n)):
            t = self.loop.create_task(self.w.run_session(uid, s, str(kw.get("agent_name", self.w.default_loop)), sp, kw, "remote"))
            self.tasks.add(t)
            t.add_done_callback(self.tasks.discard)

    def ship_finished(self) -> int:
        q = self.rb.q
        done = q.list_keys("remote", lambda k, t: t.get("kind") == "prompt" and t.get("status") in (FINISHED, FAILURE))
        for uid in done:
            keys = self.rb._group_keys(uid, "remote")
            tags = q.get_tags(uid, "remote")
            payload = {"uid": uid, "start_version": tags["start_version"], "end_version": tags.get("end_version", 0),
                       "trajs": [(k, q.get([k], None, "remote")[0], q.get_tags(k, "remote")) for k in keys]}
            self.topo.sample_qs[self.origin.pop(uid)].put(payload)
            q.delete(keys + [uid], "remote")
        return len(done)

    def inflight(self) -> int:
        return self.rb.inflight("remote")


class RolloutService:
    """Main loop of a rollout-only rank."""

    def __init__(self, config, worker, topo: SeparateTopology, tokenizer=None):
        from ....checkpoint_engine.nccl_checkpoint_engine import NCCLCheckpointEngine
        from ....workers.rollout.llm_server import LLMServerManager

        self.config, self.worker, self.topo = config, worker, topo
        self.loop = asyncio.new_event_loop()
        rc = config.actor_rollout_ref.rollout
        self.sm = self.loop.run_until_complete(LLMServerManager.create(rc, model_config=None, engines=[worker.rollout], fully_async=True))
        self.rb = ReplayBuffer("separate_async", n=int(rc.n), max_off_policy_threshold=1 << 30)
        self.version = 0
        wtq = AgentLoopWorkerTQ(config, self.sm.client(), tokenizer, None, replay_buffer=self.rb, version_fn=lambda: self.version)
        self.runner = _GroupRunner(wtq, self.rb, self.loop, topo, rc)
        self.ckpt = NCCLCheckpointEngine(group=topo.sync_group, src=0)
        self.capacity = int(rc.max_num_seqs) // max(1, int(rc.n)) + 1
        self.stats = {"groups": 0, "weight_syncs": 0}

    def _servers(self):
        return list(self.sm.servers.values())

    def _each(self, method: str, *args) -> None:
        async def go():
            await asyncio.gather(*[getattr(s, method)(*args) for s in self._servers()])

        self.loop.run_until_complete(go())

    def _sync_weights(self, version: int) -> None:
        self._each("abort_all_requests")
        self.ckpt.receive_flat(self.worker.rollout.params.flat)
        self.version = version
        self._each("clear_kv_cache")
        self._each("set_global_steps", version)
        self._each("resume_generation")
        self.stats["weight_syncs"] += 1

    def run(self, max_seconds: Optional[float] = None) -> dict:
        t0 = time.time()
        self.worker.rollout.resume_kv_cache()
        while not self.topo.stop_requested():
            v = self.topo.version()
            if v > self.version:
                self._sync_weights(v)
            while self.runner.inflight() < self.capacity:
                rec = self.topo.prompt_q.try_get(0.01)
                if rec is None:
                    break
                self.runner.submit(rec, self.version)
            self.loop.run_until_complete(asyncio.sleep(0 if self.runner.inflight() else 0.01))
            self.stats["groups"] += self.runner.ship_finished()
            if max_seconds is not None and time.time() - t0 > max_seconds:
                break
        pending = list(self.runner.tasks)
        for t in pending:
            t.cancel()

        async def go():
            await asyncio.gather(*pending, return_exceptions=True)

        self.loop.run_until_complete(go())
        return self.stats


@register_trainer("separate_async")
class PPOTrainerSeparateAsync(PPOTrainer):
    fully_async_client = True

    def __init__(self, *args, topology: Optional[SeparateTopology] = None, **kwargs):
        super().__init__(*args, **kwargs)
        self.topo = topology or SeparateTopology(0)
        self.mode = HybridEngineMode.TRAINER
        self.switch = SwitchController(enabled=bool(self._tc("hybrid_switch", True)) and self.topo.R > 0)
        self._runner: Optional[_GroupRunner] = None
        self._wait_started: Optional[float] = None
        # how many prompt groups must be ready before lent GPUs go back to training (trainer.v1.hybrid_rollout.*); it adapts
        # step by step to whether the trainer still had to wait, and is reported with the step's metrics
        from ...config.config import HybridRolloutSwitchConfig
        from .hybrid_switch import AdaptiveSwitchThreshold, SwitchCostWindow

        hc = self._tc("hybrid_rollout", None) or {}
        known = HybridRolloutSwitchConfig.__dataclass_fields__
        self.hybrid_rollout_config = HybridRolloutSwitchConfig(**{k: v for k, v in dict(hc).items() if k in known})
        self.switch_threshold = AdaptiveSwitchThreshold(self.hybrid_rollout_config, int(self.config.data.train_batch_size),
                                                        int(self._tc("parameter_sync_step", 1) or 1))
        self.switch_costs = SwitchCostWindow(self.hybrid_rollout_config.switch_cost_window_size)
        self._last_wait_s = 0.0

    # ---- set-up
    def on_init_end(self) -> None:
        if self.topo.R > 0:
            from ....checkpoint_engine.nccl_checkpoint_engine import NCCLCheckpointEngine

            self.ckpt = NCCLCheckpointEngine(group=self.topo.sync_group, src=0) if self.topo.rank == 0 else None
            self._runner = _GroupRunner(self.worker_tq, self.replay_buffer, self._loop, self.topo, self.config.actor_rollout_ref.rollout)

    # ---- producer: prompts go to the shared queue when a rollout pool exists
    def _submit_prompts(self, prompts: list[dict], partition_id: str = "train") -> int:
        if self.topo.R == 0:
            return super()._submit_prompts(prompts, partition_id)
        for p in prompts:
            uid = str(p.get("uid") or uuid.uuid4().hex)
            kw = {k: v for k, v in p.items() if not isinstance(v, torch.Tensor)}
            if "raw_prompt" not in kw and "input_ids" in p:
                ids, am = p["input_ids"], p.get("attention_mask")
                kw["raw_prompt_ids"] = (ids[am.bool()] if am is not None else ids).tolist()
            self.replay_buffer.add_prompt(uid, kw, self.param_version, partition_id)
            self.replay_buffer.mark_running(uid, partition_id)
            self.topo.prompt_q.put({"uid": uid, "kwargs": kw, "origin": self.topo.rank, "start_version": self.param_version})
        return len(prompts)

    def _target_inflight(self) -> int:
        return int(self.config.data.train_batch_size) * (1 + int(self._tc("num_warmup_batches", 1)))

    def _top_up(self) -> None:
        rb = self.replay_buffer
        if not rb.may_start_new_prompt(self.param_version):
            return
        need = self._target_inflight() - (rb.inflight() + rb.count(FINISHED) + rb.count(FAILURE))
        if need > 0:
            self._submit_prompts(self._next_prompts(need))

    # ---- consumer: drain this rank's sample queue into the local buffer
    def _drain_samples(self) -> int:
        if self.topo.R == 0:
            return 0
        got = 0
        q = self.topo.sample_qs[self.topo.rank]
        while True:
            payload = q.try_get(0.005)
            if payload is None:
                return got
            uid = payload["uid"]
            for key, fields, tags in payload["trajs"]:
                self.replay_buffer.add_trajectory(uid, tags["session"], tags["index"], fields, tags["end_version"], failed=tags["failed"])
            got += 1

    def _pump(self, seconds: float = 0.0) -> None:
        super()._pump(seconds)
        self._drain_samples()
        if self.topo.R == 0:
            return
        if self._runner is not None and self.mode is HybridEngineMode.ROLLOUT:
            while self._runner.inflight() < 2:
                rec = self.topo.prompt_q.try_get(0.005)
                if rec is None:
                    break
                self._runner.submit(rec, self.param_version)
            self._runner.ship_finished()
        elif self._wait_started is not None and self.switch.should_switch(time.time() - self._wait_started):
            self.switch_to_rollout()
        if self.mode is HybridEngineMode.TRAINER:
            time.sleep(0.002)

    # ---- hybrid switching
    def switch_to_rollout(self) -> None:
        t0 = time.time()
        self._each_server("wake_up")
        self._each_server("resume_generation")
        self.mode = HybridEngineMode.ROLLOUT
        self._switch_t0 = t0
        self.switch_costs.to_rollout.append(time.time() - t0)

    def switch_to_trainer(self) -> None:
        if self.mode is not HybridEngineMode.ROLLOUT:
            return
        t0 = time.time()
        self._each_server("abort_all_requests")  # partial outputs stay with the clients until the next switch
        super()._pump()
        self._each_server("sleep")
        self.mode = HybridEngineMode.TRAINER
        self.switch.record_switch_cost((time.time() - t0) + 0.0)
        self.switch_costs.to_trainer.append(time.time() - t0)

    # ---- hooks
    def on_train_begin(self) -> None:
        if self.topo.R == 0:
            self._each_server("wake_up")
        self._top_up()

    def on_sample_begin(self) -> None:
        self._wait_started = time.time()
        if self.topo.R == 0:
            self._each_server("resume_generation")
        self._top_up()

    def on_sample_end(self) -> None:
        self._last_wait_s = time.time() - (self._wait_started or time.time())
        self.switch.record_wait(self._last_wait_s)
        self._wait_started = None
        if self.topo.R == 0:
            self._each_server("abort_all_requests")
            super()._pump()
        else:
            self.switch_to_trainer()

    def on_step_end(self, batch, metrics, timing_raw) -> None:
        t0 = time.time()
        self._push_weights(batch, metrics, timing_raw)  # local (hybrid) engine: in place
        if self.topo.R > 0:
            if self.topo.rank == 0:
                self.topo.version(1)  # rollout ranks see the new version and join the broadcast
                actor = self.actor_rollout_wg._workers[0].actor
                self.ckpt.send_flat(actor.params.flat)
            metrics["timing_s/update_weights_remote"] = time.time() - t0
        metrics["hybrid/num_switches"] = self.switch.num_switches
        metrics["hybrid/avg_wait_s"] = self.switch.avg_wait_s
        metrics["hybrid/switch_cost_s"] = self.switch.switch_cost_s
        had_idle = self._last_wait_s > float(getattr(self.replay_buffer, "poll_interval", 0.0) or 0.0) + 1e-3
        metrics["separate_async/switch/threshold_ratio"] = self.switch_threshold.ratio
        metrics["separate_async/switch/idle"] = float(had_idle)
        self.switch_threshold.adapt(had_idle)
        metrics["separate_async/switch/threshold"] = float(self.switch_threshold.threshold())

    def shutdown(self) -> None:
        if self.topo.R > 0:
            if self.topo.trainer_group is not None:
                dist.barrier(group=self.topo.trainer_group)
            if self.topo.rank == 0:
                self.topo.stop_requested(request=True)
        super().shutdown()

    # elastic pool membership: extra engines (e.g. a trainer rank that switched) join or leave the balancer
    def add_replicas_to_balancer(self, replicas: list) -> None:
        self._loop.run_until_complete(self.server_manager.add_replicas(replicas))

    def remove_replicas_from_balancer(self, replicas: list) -> None:
        self.server_manager.lb.remove_servers([r.server_address for r in replicas])
