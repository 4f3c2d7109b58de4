"""Replay buffer between rollout and training for the v1 trainers.

Prompts are registered under key ``{uid}`` with a group status (pending -> running -> finished | failure);
trajectories under ``{uid}_{session}_{index}``. ``sample`` returns complete groups only and, before that, evicts
groups that must not be trained on:

* **DAPO filter** - all trajectories of the group have the same value of the configured reward metric (zero
  advantage signal);
* **staleness** (async modes) - the group was started more than ``max_off_policy_threshold`` weight versions
  ago: strategy ``drop`` evicts it, strategy ``wait`` never evicts but makes ``may_start_new_prompt`` return
  ``False`` while the oldest in-flight group is at the threshold so the producer stops running ahead;
* **failure** - a session raised; such groups stay sampleable by default (missing trajectories are padded
  downstream) unless ``sync_refill_failed_groups``.

Every eviction asks the trainer for replacement prompts through ``refill_fn``: ``k`` in async modes, ``2k`` for the
DAPO filter in sync mode (over-provisioning keeps the number of extra generation rounds small).

Parity target: ``verl/trainer/ppo/v1/replay_buffer.py:63-592`` (status model :80-96, eviction/refill matrix
:98-117, async variant :497).
"""

from __future__ import annotations

import time
from collections import Counter
from typing import Callable, Optional

from ....utils.transfer_queue import KVBatchMeta, TransferQueue

__all__ = ["ReplayBuffer", "ReplayBufferAsync", "PENDING", "RUNNING", "FINISHED", "FAILURE"]

PENDING, RUNNING, FINISHED, FAILURE = "pending", "running", "finished", "failure"


class ReplayBuffer:
    def __init__(self, trainer_mode: str = "sync", n: int = 1, max_off_policy_threshold: int = 1,
                 max_off_policy_strategy: str = "drop", filter_groups_metric: Optional[str] = None,
                 refill_fn: Optional[Callable[[int], None]] = None, sync_refill_failed_groups: bool = False,
                 queue: Optional[TransferQueue] = None, poll_interval: float = 0.0):
        assert max_off_policy_strategy in ("drop", "wait")
        self.mode, self.n = trainer_mode, int(n)
        self.threshold, self.strategy = int(max_off_policy_threshold), max_off_policy_strategy
        self.filter_metric = filter_groups_metric
        self.refill_fn = refill_fn
        self.refill_failed = sync_refill_failed_groups
        self.q = queue or TransferQueue()
        self.poll_interval = poll_interval
        self.metrics: Counter = Counter()
        self._staleness: list[int] = []

    @property
    def is_async(self) -> bool:
        return self.mode != "sync"

    # ---- producer side
    def add_prompt(self, uid: str, payload: dict, model_version: int, partition_id: str = "train", n: Optional[int] = None) -> None:
        """``n``: sessions that complete this prompt's group (default: the buffer's group size; validation prompts usually
        run one)."""
        self.q.put(uid, {"prompt": payload}, {"kind": "prompt", "status": PENDING, "start_version": int(model_version),
                                               "done": 0, "failed": 0, "n": int(n or self.n)}, partition_id)

    def mark_running(self, uid: str, partition_id: str = "train") -> None:
        self.q.set_tags(uid, {"status": RUNNING}, partition_id)

    def add_trajectory(self, uid: str, session: int, index: int, fields: dict, model_version: int,
                       failed: bool = False, last: bool = True, partition_id: str = "train") -> str:
        """Store one output trajectory; ``last`` marks the final trajectory of the session."""
        key = f"{uid}_{session}_{index}"
        self.q.put(key, fields, {"kind": "traj", "uid": uid, "session": session, "index": index,
                                 "end_version": int(model_version), "failed": bool(failed)}, partition_id)
        if last:
            t = self.q.get_tags(uid, partition_id)
            done, bad = t.get("done", 0) + 1, t.get("failed", 0) + int(failed)
            upd = {"done": done, "failed": bad, "end_version": max(int(model_version), t.get("end_version", 0))}
            if done >= int(t.get("n", self.n)):
                upd["status"] = FAILURE if bad else FINISHED
            self.q.set_tags(uid, upd, partition_id)
        return key

    def count(self, status: str, partition_id: str = "train") -> int:
        return len(self.q.list_keys(partition_id, lambda k, t: t.get("kind") == "prompt" and t.get("status") == status))

    def inflight(self, partition_id: str = "train") -> int:
        return self.count(PENDING, partition_id) + self.count(RUNNING, partition_id)

    def may_start_new_prompt(self, current_version: int, partition_id: str = "train") -> bool:
        """``wait`` strategy: hold the producer back while the oldest unfinished group is at the staleness limit."""
        if not self.is_async or self.strategy != "wait":
            return True
        live = self.q.list_keys(partition_id, lambda k, t: t.get("kind") == "prompt" and t.get("status") in (PENDING, RUNNING))
        oldest = min((self.q.get_tags(u, partition_id)["start_version"] for u in live), default=current_version)
        return current_version - oldest < self.threshold

    # ---- consumer side
    def _group_keys(self, uid: str, partition_id: str) -> list[str]:
        ks = self.q.list_keys(partition_id, lambda k, t: t.get("kind") == "traj" and t.get("uid") == uid)
        return sorted(ks, key=lambda k: tuple(int(x) for x in k.rsplit("_", 2)[1:]))

    def _evict(self, uid: str, partition_id: str, reason: str) -> None:
        self.q.delete(self._group_keys(uid, partition_id) + [uid], partition_id)
        self.metrics[f"replay_buffer/{reason}/evicted_groups"] += 1

    def _dapo_degenerate(self, uid: str, partition_id: str) -> bool:
        if not self.filter_metric:
            return False
        vals = []
        for rec in self.q.get(self._group_keys(uid, partition_id), ["reward_extra_info", self.filter_metric], partition_id):
            info = rec.get("reward_extra_info") or {}
            vals.append(info.get(self.filter_metric, rec.get(self.filter_metric)))
        return len(vals) > 0 and all(v == vals[0] for v in vals)

    def _sweep(self, current_version: int, partition_id: str, validate: bool) -> list[str]:
        """Apply the eviction rules to all terminal groups; returns the uids that may be trained on."""
        terminal = self.q.list_keys(partition_id, lambda k, t: t.get("kind") == "prompt" and t.get("status") in (FINISHED, FAILURE))
        ok, refill = [], 0
        for uid in terminal:
            t = self.q.get_tags(uid, partition_id)
            if validate:
                ok.append(uid)
                continue
            age = current_version - t["start_version"]
            if self.is_async and self.strategy == "drop" and age > self.threshold:
                self._staleness.append(age)
                self._evict(uid, partition_id, "off_policy")
                refill += 1
            elif t["status"] == FAILURE and (self.is_async or self.refill_failed) and not self._group_keys(uid, partition_id):
                self._evict(uid, partition_id, "failure")
                refill += 1
            elif self._dapo_degenerate(uid, partition_id):
                self._evict(uid, partition_id, "dapo")
                refill += 1 if self.is_async else 2
            else:
                ok.append(uid)
        if refill and self.refill_fn is not None:
            self.metrics["replay_buffer/refill_prompts"] += refill
            self.refill_fn(refill)
        return sorted(ok, key=lambda u: (self.q.get_tags(u, partition_id)["start_version"], u))

    def ready(self, num_prompts: int, current_version: int = 0, partition_id: str = "train", validate: bool = False) -> bool:
        return len(self._sweep(current_version, partition_id, validate)) >= num_prompts

    def sample(self, num_prompts: int, current_version: int = 0, partition_id: str = "train", validate: bool = False,
               timeout: Optional[float] = None, pump: Optional[Callable[[], None]] = None) -> Optional[KVBatchMeta]:
        """Oldest-first ``num_prompts`` complete groups as a key handle (the groups leave the buffer's bookkeeping;
        call ``release`` after training). ``pump`` is called between polls (drives an in-process producer)."""
        t0 = time.time()
        while True:
            ok = self._sweep(current_version, partition_id, validate)
            if len(ok) >= num_prompts:
                break
            if self.inflight(partition_id) == 0 and pump is None:
                return None  # nothing will ever arrive
            if timeout is not None and time.time() - t0 > timeout:
                return None
            if pump is not None:
                pump()
            elif self.poll_interval:
                time.sleep(self.poll_interval)
        chosen = ok[:num_prompts]
        keys: list[str] = []
        for uid in chosen:
            keys += self._group_keys(uid, partition_id)
            t = self.q.get_tags(uid, partition_id)
            self._staleness.append(current_version - t["start_version"])
            self.q.set_tags(uid, {"status": "sampled"}, partition_id)
        self.metrics["replay_buffer/sampled_groups"] += len(chosen)
        meta = self.q.get_meta(keys, None, partition_id)
        meta.uids = chosen  # type: ignore[attr-defined]
        return meta

    def release(self, meta: KVBatchMeta) -> None:
        self.q.delete(list(meta.keys) + list(getattr(meta, "uids", [])), meta.partition_id)

    def drain_inflight(self, partition_id: str = "train") -> int:
        """Sync mode after sampling: whatever is still pending/running/terminal belongs to no future step."""
        rest = self.q.list_keys(partition_id, lambda k, t: t.get("kind") == "prompt" and t.get("status") != "sampled")
        for uid in rest:
            self._evict(uid, partition_id, "drained")
        return len(rest)

    def pop_metrics(self) -> dict:
        out = dict(self.metrics)
        if self._staleness:
            s = self._staleness
            out.update({"replay_buffer/staleness/mean": sum(s) / len(s), "replay_buffer/staleness/max": max(s),
                        "replay_buffer/staleness/min": min(s)})
        self.metrics.clear()
        self._staleness = []
        return out


class ReplayBufferAsync(ReplayBuffer):
    """Async-mode defaults (``k`` evictions -> ``k`` refills; staleness rules active)."""

    def __init__(self, *args, **kwargs):
        kwargs.setdefault("trainer_mode", "colocate_async")
        super().__init__(*args, **kwargs)
