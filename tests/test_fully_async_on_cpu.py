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
    assert m == {"a/max": 3.0, "a/mean": 3.25, "timing_s/gen": 3.0}
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
