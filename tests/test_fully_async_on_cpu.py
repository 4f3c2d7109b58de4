"""Fully-async pipeline: queue semantics, staleness pause, schedule policies, and two training steps on CPU."""
import pytest

from verl_b200.experimental.fully_async_policy.detach_utils import MetricsAggregator
from verl_b200.experimental.fully_async_policy.dynamic_schedule import (DefaultDynamicSchedulePolicy, DynamicResourceController,
                                                                        FixedRatioDynamicSchedulePolicy, StaticFullyAsyncPolicy)
from verl_b200.experimental.fully_async_policy.message_queue import MessageQueue


def test_message_queue_bounds_and_staleness():
    q = MessageQueue(max_queue_size=2, staleness_threshold=1)
    assert q.put_sample("a", 0) and q.put_sample("b", 0) and q.put_sample("c", 0)  # "a" is dropped
    assert q.get_sample(0)[0] == "b" and q.get_statistics()["dropped_samples"] == 1
    q.update_param_version(3)
    assert not q.put_sample("stale", 1) and q.put_sample("fresh", 2)
    assert q.get_sample(0)[0] == "c" and q.get_sample(0)[0] == "fresh" and q.get_sample(0) is None
    q.shutdown()
    assert not q.put_sample("x", 3)


def test_metrics_aggregator_and_schedule_policies():
    agg = MetricsAggregator()
    agg.add_step_metrics({"a/mean": 1.0, "a/max": 1.0, "timing_s/gen": 2.0}, 1)
    agg.add_step_metrics({"a/mean": 4.0, "a/max": 3.0, "timing_s/gen": 1.0}, 3)
    m = agg.get_aggregated_metrics()
    assert m == {"a/max": 3.0, "a/mean": 2.5, "timing_s/gen": 3.0}  # plain mean over steps; weighting is opt-in by name
    log = []
    c = DynamicResourceController(DefaultDynamicSchedulePolicy(), elastic=2, add_fn=lambda k: log.append(+k), remove_fn=lambda k: log.append(-k))
    assert c.step(queue_size=0, required_samples=8, trainer_idle_s=5, trainer_step_s=5) == 1
    assert c.step(0, 8, 5, 5) == 2 and c.step(0, 8, 5, 5) == 2
    assert c.step(queue_size=40, required_samples=8, trainer_idle_s=0.0, trainer_step_s=10) == 1
    assert log == [1, 1, -1]
    assert DynamicResourceController(StaticFullyAsyncPolicy(), 4).step(0, 8, 9, 1) == 0
    assert DynamicResourceController(FixedRatioDynamicSchedulePolicy(0.5), 4).step(0, 8, 1, 1) == 2


def test_fully_async_trains_and_respects_staleness_budget(monkeypatch):
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    from tests.test_v1_trainer_on_cpu import ARGS
    from verl_b200.experimental.fully_async_policy.fully_async_main import main

    t = main(ARGS + ["+async_training.require_batches=1", "+async_training.trigger_parameter_sync_step=2",
                     "+async_training.staleness_threshold=0.5", "trainer.total_training_steps=4"])
    assert t.param_version == 2 and t.local_updates == 4
    r = t.rollouter
    assert r.max_samples_per_version() == 12  # 4 samples x 2 updates x (1 + 0.5)
    assert r.produced >= 16 and r.stats["pauses"] >= 1
    assert r.produced <= 16 + r.max_samples_per_version()  # never ran ahead by more than one budget
    # the cycle's aggregated record: summed seconds, one utilisation ratio per side and the combined figure
    agg = t.last_aggregated_metrics
    assert 0.0 < agg["dynamic_resource/train_resource_utilization"] <= 1.0
    assert 0.0 <= agg["dynamic_resource/rollout_resource_utilization"] <= 1.0
    assert 0.0 <= agg["dynamic_resource/resource_utilization"] <= 1.0
    assert abs(agg["fully_async/trainer/idle_ratio"] - agg["timing_s/gen"] / agg["timing_s/step"]) < 1e-9
    assert agg["fully_async/param_version"] == 2 and agg["training/global_step"] == 4


def test_metrics_aggregator_reduces_by_name_and_derives_cycle_figures():
    from verl_b200.experimental.fully_async_policy.detach_utils import MetricsAggregator

    a = MetricsAggregator(total_gpus=4, hybrid_gpus=2, standalone_gpus=2)
    assert a.get_aggregated_metrics() == {}
    rule = MetricsAggregator.rule
    assert rule("timing_s/gen") == "sum" and rule("timing_s/agent_loop/tool_calls/max") == "max" and rule("perf/time_per_step") == "sum"
    assert rule("critic/score/mean") == "mean" and rule("response_length/max") == "max" and rule("prompt_length/min") == "min"
    assert rule("perf/total_num_tokens") == "sum" and rule("training/global_step") == "last" and rule("actor/pg_loss") == "mean"
    assert rule("x/weighted_avg_thing") == "weighted"
    steps = [
        {"timing_s/step": 10.0, "timing_s/gen": 4.0, "timing_s/wait_for_enough_samples": 4.0, "perf/time_per_step": 10.0,
         "perf/total_num_tokens": 4000, "perf/throughput": 1.0, "critic/score/mean": 0.2, "response_length/max": 50,
         "global_seqlen/max": 900, "global_seqlen/min": 300, "global_seqlen/minmax_diff": 1, "training/global_step": 7,
         "dynamic_resource/train_compute_time_s": 5.0, "dynamic_resource/train_allocated_time_s": 6.0, "x/weighted_avg_thing": 1.0,
         "flag": True, "text": "ignored", "tensor": __import__("torch").tensor(2.0)},
        {"timing_s/step": 30.0, "timing_s/gen": 6.0, "timing_s/wait_for_enough_samples": 6.0, "perf/time_per_step": 30.0,
         "perf/total_num_tokens": 12000, "perf/throughput": 2.0, "critic/score/mean": 0.4, "response_length/max": 70,
         "global_seqlen/max": 800, "global_seqlen/min": 200, "global_seqlen/minmax_diff": 1, "training/global_step": 8,
         "dynamic_resource/train_compute_time_s": 13.0, "dynamic_resource/train_allocated_time_s": 24.0, "x/weighted_avg_thing": 4.0,
         "tensor": __import__("torch").tensor(4.0)},
    ]
    a.add_step_metrics(steps[0], sample_count=1)
    a.add_step_metrics(steps[1], sample_count=3)
    assert a.get_current_stats()["step_count"] == 2 and a.get_current_stats()["total_samples"] == 4
    out = a.get_aggregated_metrics(rollout_resource_utilization=0.5)
    assert out["timing_s/step"] == 40.0 and out["critic/score/mean"] == pytest.approx(0.3) and out["response_length/max"] == 70
    assert out["training/global_step"] == 8 and out["x/weighted_avg_thing"] == pytest.approx(3.25) and out["tensor"] == 3.0
    assert "flag" not in out and "text" not in out
    assert out["global_seqlen/minmax_diff"] == 900 - 200
    assert out["perf/throughput"] == pytest.approx(16000 / (40.0 * 4))
    assert out["fully_async/trainer/idle_ratio"] == pytest.approx(0.25)
    u_train = 18.0 / 30.0
    assert out["dynamic_resource/train_resource_utilization"] == pytest.approx(u_train)
    x = 10.0 / 40.0
    assert out["dynamic_resource/resource_utilization"] == pytest.approx(((1 - x) * 2 * u_train + (x * 2 + 2) * 0.5) / 4)
    # without the rollouter's figure the combined one is not reported
    assert "dynamic_resource/resource_utilization" not in a.get_aggregated_metrics()
    a.reset()
    assert a.step_count == 0 and a.get_aggregated_metrics() == {}


def test_safe_create_task_keeps_and_reports_background_tasks(caplog):
    import asyncio
    import logging

    from verl_b200.experimental.fully_async_policy.detach_utils import safe_create_task

    async def ok():
        return 1

    async def boom():
        raise RuntimeError("lost replica")

    async def main():
        held = set()
        a = safe_create_task(ok(), "fine", held)
        b = safe_create_task(boom(), "broken", held)
        assert held == {a, b}
        await asyncio.gather(a, b, return_exceptions=True)
        await asyncio.sleep(0)
        return held

    with caplog.at_level(logging.ERROR):
        loop = asyncio.new_event_loop()
        try:
            asyncio.set_event_loop(loop)
            held = loop.run_until_complete(main())
        finally:
            asyncio.set_event_loop(None)
            loop.close()
    assert held == set() and any("broken" in r.getMessage() and "lost replica" in r.getMessage() for r in caplog.records)


class _StepServer:
    """A rollout server stand-in: emits one token per tick; the token is 1000 * weight_version + position, so a sequence
    shows which weights produced each of its tokens. ``abort_all_requests`` ends every running call with what it has."""

    def __init__(self, name):
        self.name, self.version, self.running, self.calls, self.paused = name, 0, {}, 0, False
        self._abort = 0

    async def generate(self, prompt_ids, sampling_params, request_id, **kw):
        import asyncio

        from verl_b200.workers.rollout.replica import TokenOutput

        self.calls += 1
        self.running[request_id] = True
        epoch = self._abort
        out = []
        try:
            while len(out) < sampling_params["max_tokens"]:
                await asyncio.sleep(0.001)
                if self._abort != epoch:
                    return TokenOutput(out, [0.0] * len(out), None, "aborted")
                while self.paused:
                    await asyncio.sleep(0.001)
                out.append(1000 * self.version + len(prompt_ids) + len(out))
            return TokenOutput(out, [0.0] * len(out), None, "length")
        finally:
            self.running.pop(request_id, None)

    async def abort_all_requests(self):
        self._abort += 1
        self.paused = True

    async def resume_generation(self):
        self.paused = False


class _Replica:
    def __init__(self, name):
        self.server_address, self.server_handle = name, _StepServer(name)

    async def abort_all_requests(self):
        await self.server_handle.abort_all_requests()


def _manager(replicas, response_length=40):
    from verl_b200.workers.rollout.llm_server import LLMServerManager

    return LLMServerManager({"prompt_length": 8, "response_length": response_length}, replicas, fully_async=True)


def test_partial_rollout_resumes_under_new_weights():
    """A weight update aborts what runs; the client keeps the tokens made so far and the same request continues with the
    new weights for the rest of its budget: no token is generated twice and none is lost."""
    import asyncio

    async def go():
        rep = _Replica("r0")
        sm = _manager([rep])
        client = sm.client()
        task = asyncio.ensure_future(client.generate("req", prompt_ids=[1, 2, 3], sampling_params={"max_tokens": 30}))
        await asyncio.sleep(0.015)
        # parameter sync: abort, install version 1, resume
        await rep.server_handle.abort_all_requests()
        rep.server_handle.version = 1
        await rep.server_handle.resume_generation()
        out = await task
        return out, rep.server_handle.calls

    out, calls = asyncio.run(go())
    assert len(out.token_ids) == 30 and out.stop_reason == "length" and calls == 2
    versions = [t // 1000 for t in out.token_ids]
    cut = versions.index(1)
    assert 0 < cut < 30 and versions == [0] * cut + [1] * (30 - cut)          # old-weight prefix, new-weight rest
    assert [t % 1000 for t in out.token_ids] == list(range(3, 33))             # contiguous positions: nothing redone or dropped
    assert out.num_preempted == 1


def test_rebalance_moves_inflight_requests_to_added_replicas():
    import asyncio

    from verl_b200.experimental.fully_async_policy.fully_async_rollouter import FullyAsyncRollouter
    from verl_b200.experimental.fully_async_policy.message_queue import MessageQueue

    async def go():
        r0 = _Replica("r0")
        sm = _manager([r0], response_length=400)
        client = sm.client()
        roll = FullyAsyncRollouter(agent_worker=None, server_manager=sm, message_queue=MessageQueue(8, 1), prompt_source=lambda k: [],
                                   n=1, sampling_params={}, required_samples=4, max_queue_size=2)
        tasks = [asyncio.ensure_future(client.generate(f"q{i}", prompt_ids=[1], sampling_params={"max_tokens": 300})) for i in range(8)]
        await asyncio.sleep(0.01)
        assert sm.lb.snapshot() == {"r0": 8}
        r1, r2, r3 = _Replica("r1"), _Replica("r2"), _Replica("r3")
        await roll.add_replicas([r1, r2, r3])
        assert sm.lb.snapshot() == {"r0": 8, "r1": 0, "r2": 0, "r3": 0}      # sticky: nothing moves by itself
        diag = await roll.rebalance_requests()
        await asyncio.sleep(0.08)                                                # retries land (client retry interval 0.05 s)
        loads = sm.lb.snapshot()
        outs = await asyncio.gather(*tasks)
        return diag, loads, outs, roll

    diag, loads, outs, roll = asyncio.run(go())
    assert diag["cleared_entries"] == 8 and diag["inflight_after_wait"] == 0 and roll.stats["rebalances"] == 1
    assert sorted(loads.values()) == [2, 2, 2, 2], loads
    assert all(len(o.token_ids) == 300 and [t % 1000 for t in o.token_ids] == list(range(1, 301)) for o in outs)


def test_rollouter_pauses_on_a_full_queue():
    from verl_b200.experimental.fully_async_policy.fully_async_rollouter import FullyAsyncRollouter
    from verl_b200.experimental.fully_async_policy.message_queue import MessageQueue

    q = MessageQueue(8, 1)
    roll = FullyAsyncRollouter(agent_worker=None, server_manager=None, message_queue=q, prompt_source=lambda k: [{"x": 1}], n=1,
                               sampling_params={}, required_samples=100, max_queue_size=2)
    assert not roll._should_pause_generation()
    q.put_sample("a", 0)
    q.put_sample("b", 0)
    assert roll._should_pause_generation() and roll.stats["pause_reason"] == "queue_full"
    q.get_sample(0)
    assert not roll._should_pause_generation()


def test_rollouter_step_accounting_and_capacity_utilisation():
    """The producer's step record after a weight sync: utilisation is the time-weighted share of the capacity in use, with
    the capacity that held during each interval (replicas come and go inside a step); idle time starts when production
    ran dry; the concurrency limit follows the number of replicas."""
    import time

    from verl_b200.experimental.fully_async_policy.fully_async_rollouter import FullyAsyncRollouter
    from verl_b200.experimental.fully_async_policy.message_queue import MessageQueue

    class SM:
        replicas = [object(), object()]

    r = FullyAsyncRollouter(agent_worker=None, server_manager=SM(), message_queue=MessageQueue(64), prompt_source=lambda k: [],
                            n=1, sampling_params={}, required_samples=4, max_concurrent_samples=8)
    t0 = 1000.0
    # 2 s with 4 of 8 busy, 1 s with 8 of 16 after two replicas joined, 1 s with 20 of 16 (clamped), 1 s without capacity
    r._active_history = [(t0, 4, 8), (t0 + 2, 8, 16), (t0 + 3, 20, 16), (t0 + 4, 3, 0), (t0 + 5, 0, 8)]
    real_time = time.time
    try:
        time.time = lambda: t0 + 5
        u = r._compute_rollout_resource_utilization()
    finally:
        time.time = real_time
    assert abs(u - (2 * 4 + 1 * 8 + 1 * 16) / (2 * 8 + 1 * 16 + 1 * 16)) < 1e-9
    assert len(r._active_history) == 1

    assert r._per_replica == 4.0
    SM.replicas = [object()] * 3
    r._update_max_concurrent_samples()
    assert r.max_concurrent == 12
    r._step_generated, r._step_start = 5, real_time() - 2.0
    r._idle_start = r._step_start + 0.5                        # production ran dry half a second into the step
    rec = r.reset_staleness()
    assert rec["fully_async/rollouter/step_generated_samples"] == 5 and r.completed_steps == 1 and r._step_generated == 0
    assert abs(rec["fully_async/rollouter/active_time"] - 0.5) < 1e-6 and 0.7 < rec["fully_async/rollouter/idle_ratio"] < 0.8
    assert 0.0 <= rec["dynamic_resource/rollout_resource_utilization"] <= 1.0 and r.step_samples_history == [(1, 5)]
    assert r.statistics()["rollouter/max_concurrent_samples"] == 12


def test_fully_async_checkpoint_keeps_queued_samples_and_inflight_prompts(monkeypatch, tmp_path):
    """A run saves at the end of a synchronisation cycle; a second run resumes from it with the producer's counters, the
    samples that were queued for the trainer and the prompts that were in flight (re-issued before any new prompt)."""
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    import os

    import torch

    from tests.test_v1_trainer_on_cpu import ARGS
    from verl_b200.experimental.fully_async_policy.fully_async_main import main

    base = [a for a in ARGS if not a.startswith(("trainer.resume_mode", "trainer.total_training_steps"))] + [
        "+async_training.require_batches=1", "+async_training.trigger_parameter_sync_step=1", "+async_training.staleness_threshold=1.0",
        f"trainer.default_local_dir={tmp_path}", "trainer.save_freq=2"]
    base[-1] = "trainer.save_freq=1"
    t1 = main(base + ["trainer.total_training_steps=1", "trainer.resume_mode=disable"])
    folder = os.path.join(str(tmp_path), "global_step_1")
    path = os.path.join(folder, "rollouter.pt")
    sd = torch.load(path, weights_only=False)
    own = torch.load(os.path.join(folder, "fully_async_trainer.pt"), weights_only=False)
    assert own == {"local_updates": 1, "param_version": 1} and sd["param_version"] == 1
    # the producer ran ahead of the trainer: eight groups were admitted, four were trained on, four wait in the queue
    assert sd["produced"] == 8 and len(sd["queued"]) == 4 and sd["inflight_prompts"] == []
    # make one of the queued groups an in-flight prompt instead, as if the checkpoint had caught it mid-generation
    moved, _ = sd["queued"].pop()
    sd["inflight_prompts"] = [dict(moved.prompt)]
    sd["produced"] -= 1
    torch.save(sd, path)
    queued_ids = [s.sample_id for s, _ in sd["queued"]]
    inflight_uids = [p["uid"] for p in sd["inflight_prompts"]]
    assert len(queued_ids) == 3 and inflight_uids == [moved.uid]

    # resume: look at the restored state before any training happens
    from verl_b200.experimental.fully_async_policy import fully_async_trainer as fat

    seen = {}
    orig = fat.FullyAsyncTrainer._load_checkpoint

    def spy(self):
        step = orig(self)
        seen.update(step=step, queued=[s.sample_id for s, _ in self.mq.snapshot()], replay=[p["uid"] for p in self.rollouter._replay],
                    version=self.rollouter.param_version, local_updates=self.local_updates, produced=self.rollouter.produced,
                    since_sync=self.rollouter.produced_since_sync)
        return step

    monkeypatch.setattr(fat.FullyAsyncTrainer, "_load_checkpoint", spy)
    t2 = main(base + ["trainer.total_training_steps=2", "trainer.resume_mode=auto"])
    assert seen["step"] == 1 and seen["queued"] == queued_ids and seen["replay"] == inflight_uids
    assert seen["version"] == 1 and seen["local_updates"] == 1 and seen["produced"] == sd["produced"]
    assert seen["since_sync"] == len(queued_ids)
    assert t2.global_steps == 3 and t2.param_version == 2 and t2.local_updates == 2
    # the fourth sample of the resumed step came from the re-issued prompt, admitted before any new one and not counted twice
    assert not t2.rollouter._replay and t2.rollouter.produced == sd["produced"] + (t2.rollouter.submitted - sd["submitted"]) + 1
    assert moved.uid in [u for u in t2.last_batch.non_tensor_batch["uid"]]
