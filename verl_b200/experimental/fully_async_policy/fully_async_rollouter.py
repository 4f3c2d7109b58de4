"""Streaming sample producer of the fully-asynchronous pipeline.

Owns the prompt stream. Keeps up to ``max_concurrent_samples`` prompts in flight on the rollout replicas, packs each
finished group into a ``RolloutSample`` and puts it on the message queue. Production pauses while the number of
samples that would be stale when consumed reaches the budget
``required_samples x trigger_parameter_sync_step x (1 + staleness_threshold)`` counted since the last weight sync
(finished-but-unconsumed + in flight), and resumes after the next sync. Replicas can be added, removed and
rebalanced while requests are running.

After every weight sync ``reset_staleness`` closes the producer's "step": it reports how long the replicas were busy and
idle since the previous sync, how many groups were produced, and the time-weighted utilisation of the rollout capacity
(which changes when replicas come and go).

Parity target: ``verl/experimental/fully_async_policy/fully_async_rollouter.py`` (``_compute_rollout_resource_utilization``
:536, ``reset_staleness`` :594, ``_feed_samples`` :859, ``_record_active_count`` :892, ``_processor_worker`` :902,
``_streaming_generation_main`` :1017, ``_should_pause_generation`` :1142, ``add_replicas/remove_replicas/rebalance_requests``
:144-264, :1199-1274, ``_update_max_concurrent_samples`` :1274).
"""

from __future__ import annotations

import asyncio
import time
import uuid
from typing import Callable, Iterator, Optional

from .detach_utils import RolloutSample
from .message_queue import MessageQueue

__all__ = ["FullyAsyncRollouter"]


class FullyAsyncRollouter:
    def __init__(self, agent_worker, server_manager, message_queue: MessageQueue, prompt_source: Callable[[int], list[dict]],
                 n: int, sampling_params: dict, required_samples: int, trigger_parameter_sync_step: int = 1,
                 staleness_threshold: float = 1.0, max_concurrent_samples: Optional[int] = None, total_samples: Optional[int] = None,
                 max_queue_size: Optional[int] = None):
        self.w, self.sm, self.mq = agent_worker, server_manager, message_queue
        self.prompt_source, self.n, self.sp = prompt_source, int(n), dict(sampling_params)
        self.required_samples = int(required_samples)
        self.trigger = max(1, int(trigger_parameter_sync_step))
        self.staleness_threshold = float(staleness_threshold)
        self.max_concurrent = int(max_concurrent_samples or 2 * required_samples)
        self.total_samples = total_samples
        # finished samples waiting for the trainer: production also stops while the queue is full (nothing would be gained
        # by producing samples that push older ones out)
        self.max_queue_size = int(max_queue_size) if max_queue_size else None
        self.param_version = 0
        self.submitted = self.produced = self.produced_since_sync = 0
        self.paused = False
        self.running: dict[str, asyncio.Task] = {}
        self._inflight_prompts: dict[str, dict] = {}   # what ``running`` was started from: a checkpoint re-issues these
        self._replay: list[dict] = []                  # prompts restored from a checkpoint, served before new ones
        self.stats = {"pauses": 0, "failed": 0}
        # bookkeeping of the producer's step (the span between two weight syncs)
        self._per_replica = self.max_concurrent / max(1, self._num_replicas())  # concurrency one replica is worth
        self._active_history: list[tuple[float, int, int]] = [(time.time(), 0, self.max_concurrent)]
        self._step_start = time.time()
        self._idle_start = 0.0          # when production last ran dry (paused with nothing in flight)
        self._step_generated = 0
        self.completed_steps = 0
        self.step_samples_history: list[tuple[int, int]] = []

    # ---- staleness control
    def max_samples_per_version(self) -> int:
        return int(self.required_samples * self.trigger * (1.0 + self.staleness_threshold))

    def _should_pause_generation(self) -> bool:
        if self.total_samples is not None and self.submitted >= self.total_samples:
            return True
        if self.max_queue_size is not None and self.mq.get_queue_size() >= self.max_queue_size:
            self.stats["pause_reason"] = "queue_full"
            return True
        if self.produced_since_sync + len(self.running) >= self.max_samples_per_version():
            self.stats["pause_reason"] = "staleness"
            return True
        return False

    def update_param_version(self, version: int) -> dict:
        """Called by the parameter synchroniser after a weight sync: the budget starts over. Returns the timing record of
        the step that ended (``reset_staleness``)."""
        self.param_version = int(version)
        return self.reset_staleness()

    # ---- utilisation of the rollout capacity
    def _num_replicas(self) -> int:
        return len(getattr(self.sm, "replicas", None) or []) or 1

    def _record_active_count(self) -> None:
        """Event-driven history (time, trajectories groups in flight, capacity): one entry whenever either number changes."""
        self._active_history.append((time.time(), len(self.running), self.max_concurrent))

    def _update_max_concurrent_samples(self) -> None:
        """The concurrency limit follows the number of active replicas (each replica is worth what it was worth at start)."""
        self.max_concurrent = max(1, int(round(self._per_replica * self._num_replicas())))
        self._record_active_count()

    def _compute_rollout_resource_utilization(self) -> float:
        """Share of the rollout capacity that was in use since the previous call: with the history entries (t_k, A_k, S_k),
        sum_k (t_{k+1} - t_k) * min(A_k, S_k) / sum_k (t_{k+1} - t_k) * S_k. Every interval uses the capacity that held
        during it (replicas can come and go inside a step); intervals without capacity carry no weight."""
        self._record_active_count()
        num = den = 0.0
        for (t0, active, cap), (t1, _, _) in zip(self._active_history, self._active_history[1:]):
            dt = t1 - t0
            if dt <= 0 or cap <= 0:
                continue
            num += dt * min(active, cap)
            den += dt * cap
        self._active_history = [self._active_history[-1]]
        return num / den if den > 0 else 0.0

    def reset_staleness(self) -> dict:
        """After a weight sync: what is still queued or in flight was started under older weights and counts against the
        new budget; production resumes. Returns the producer-side timing of the step that ended."""
        self.paused = False
        self.produced_since_sync = self.mq.get_queue_size()
        now = time.time()
        span = max(now - self._step_start, 1e-6)
        active = self._idle_start - self._step_start if self._idle_start > self._step_start else span
        timing = {"fully_async/rollouter/active_time": active, "fully_async/rollouter/version_time": span,
                  "fully_async/rollouter/idle_ratio": 1.0 - active / span,
                  "fully_async/rollouter/step_generated_samples": self._step_generated,
                  "dynamic_resource/rollout_resource_utilization": self._compute_rollout_resource_utilization()}
        if self._step_generated > 0:
            self.completed_steps += 1
            self.step_samples_history = (self.step_samples_history + [(self.completed_steps, self._step_generated)])[-16:]
        self._step_generated = 0
        self._step_start = now
        return timing

    # ---- production
    async def _one_sample(self, prompt: dict) -> None:
        uid = str(prompt.get("uid") or uuid.uuid4().hex)
        t0, v0 = time.time(), self.param_version
        name = str(prompt.get("agent_name", self.w.default_loop))
        outs = await asyncio.gather(*[self.w._run_one(name, self.sp, prompt) for _ in range(self.n)], return_exceptions=True)
        bad = [o for o in outs if isinstance(o, BaseException)]
        good = [o for o in outs if not isinstance(o, BaseException)]
        self.stats["failed"] += len(bad)
        sample = RolloutSample(sample_id=f"{uid}@{v0}", uid=uid, trajectories=good, prompt=prompt, param_version_start=v0,
                               param_version_end=self.param_version, processing_time=time.time() - t0, failed=bool(bad))
        self.running.pop(uid, None)
        self._inflight_prompts.pop(uid, None)
        self._record_active_count()
        if good:
            self.mq.put_sample(sample, self.param_version)
            self.produced += 1
            self.produced_since_sync += 1
            self._step_generated += 1

    def feed(self) -> int:
        """Admit prompts up to the concurrency and staleness limits; returns how many were started."""
        started = 0
        while len(self.running) < self.max_concurrent:
            if self._should_pause_generation():
                if not self.paused:
                    self.paused = True
                    self.stats["pauses"] += 1
                if not self.running and self._idle_start <= self._step_start:
                    self._idle_start = time.time()   # nothing in flight and nothing may start: the replicas idle from here
                break
            resumed = bool(self._replay)
            got = [self._replay.pop(0)] if resumed else self.prompt_source(1)
            if not got:
                break
            p = dict(got[0])
            p.setdefault("uid", uuid.uuid4().hex)
            self._inflight_prompts[p["uid"]] = p
            self.running[p["uid"]] = asyncio.ensure_future(self._one_sample(p))
            self.submitted += 0 if resumed else 1   # a re-issued prompt was counted when it was first admitted
            started += 1
        if started:
            self._record_active_count()
        return started

    # ---- checkpoint
    def state_dict(self) -> dict:
        """Everything a resumed run needs to lose no prompt: the counters, the finished samples still queued for the trainer
        and the prompts whose trajectories were being generated (their partial output is not kept: they start again).
        The reference saves the dataloader position only and loses both kinds
        (``verl/experimental/fully_async_policy/fully_async_rollouter.py:655-670``)."""
        return {"param_version": self.param_version, "submitted": self.submitted, "produced": self.produced,
                "produced_since_sync": self.produced_since_sync, "completed_steps": self.completed_steps,
                "stats": dict(self.stats), "step_samples_history": list(self.step_samples_history),
                "inflight_prompts": [dict(p) for p in self._inflight_prompts.values()] + [dict(p) for p in self._replay],
                "queued": self.mq.snapshot()}

    def load_state_dict(self, sd: dict) -> None:
        self.param_version = int(sd.get("param_version", 0))
        self.submitted, self.produced = int(sd.get("submitted", 0)), int(sd.get("produced", 0))
        self.completed_steps = int(sd.get("completed_steps", 0))
        self.stats.update(sd.get("stats", {}))
        self.step_samples_history = [tuple(x) for x in sd.get("step_samples_history", [])]
        self.mq.restore(sd.get("queued", []))
        # queued samples were produced under older weights: they count against the staleness budget of the resumed version
        self.produced_since_sync = self.mq.get_queue_size()
        self._replay = [dict(p) for p in sd.get("inflight_prompts", [])]
        self.paused = False

    def save_checkpoint(self, folder: str) -> str:
        import os

        import torch

        os.makedirs(folder, exist_ok=True)
        path = os.path.join(folder, "rollouter.pt")
        torch.save(self.state_dict(), path)
        return path

    def load_checkpoint(self, folder: str) -> bool:
        import os

        import torch

        path = os.path.join(folder, "rollouter.pt")
        if not os.path.exists(path):
            return False
        self.load_state_dict(torch.load(path, map_location="cpu", weights_only=False))
        return True

    async def run(self, stop: Callable[[], bool], idle_sleep: float = 0.0) -> None:
        """Streaming main loop (for a dedicated event loop / thread)."""
        while not stop():
            self.feed()
            await asyncio.sleep(idle_sleep)

    # ---- elastic replicas
    async def add_replicas(self, replicas: list) -> None:
        await self.sm.add_replicas(replicas)
        self._update_max_concurrent_samples()

    async def remove_replicas(self, replicas: list) -> None:
        """Stop routing to the replicas, abort what they run (clients re-issue elsewhere with the partial output)."""
        self.sm.lb.remove_servers([r.server_address for r in replicas])
        for r in replicas:
            await r.server_handle.abort_all_requests()
            await r.server_handle.resume_generation()
            self.sm.servers.pop(r.server_address, None)
            if r in self.sm.replicas:
                self.sm.replicas.remove(r)
        self._update_max_concurrent_samples()

    async def rebalance_requests(self, wait_inflight_timeout_s: float = 30.0, wait_inflight_poll_interval_s: float = 0.01) -> dict:
        """Spread the requests in flight evenly over the replicas that are active now (after replicas were added, the old
        ones carry everything and the new ones nothing): (1) forget the sticky request -> server map, (2) abort what every
        replica runs (the clients keep the partial outputs and re-issue the rest), (3) wait until the aborted calls have
        released their servers, so that the counts the router sees are true, (4) let the replicas generate again: the
        retries go to the least-loaded replicas. Returns the diagnostics of step 1 plus what was still in flight at the
        end of step 3. Parity target: ``fully_async_rollouter.py:1211-1274``."""
        result = self.sm.lb.clear_sticky_cache()
        replicas = list(self.sm.replicas)
        if replicas:
            await asyncio.gather(*[r.server_handle.abort_all_requests() for r in replicas])
        deadline = time.time() + wait_inflight_timeout_s
        while self.sm.lb.get_total_inflight() > 0 and time.time() < deadline:
            await asyncio.sleep(wait_inflight_poll_interval_s)
        result["inflight_after_wait"] = self.sm.lb.get_total_inflight()
        if replicas:
            await asyncio.gather(*[r.server_handle.resume_generation() for r in replicas])
        self.stats["rebalances"] = self.stats.get("rebalances", 0) + 1
        return result

    def statistics(self) -> dict:
        return {"rollouter/submitted": self.submitted, "rollouter/produced": self.produced, "rollouter/running": len(self.running),
                "rollouter/pauses": self.stats["pauses"], "rollouter/failed_sessions": self.stats["failed"],
                "rollouter/param_version": self.param_version, "rollouter/queue_size": self.mq.get_queue_size(),
                "rollouter/max_concurrent_samples": self.max_concurrent, "rollouter/completed_steps": self.completed_steps,
                "rollouter/paused": int(self.paused)}
