"""v1 replay buffer: group completion, DAPO filter + refill credits, staleness drop / wait, failure groups."""
from verl_b200.trainer.ppo.v1.replay_buffer import FAILURE, FINISHED, ReplayBuffer, ReplayBufferAsync


def _fill(rb, uid, n, version, metric=None, fail_session=None):
    rb.add_prompt(uid, {"q": uid}, version)
    rb.mark_running(uid)
    for s in range(n):
        rb.add_trajectory(uid, s, 0, {"response_ids": [s], "reward_extra_info": {"acc": (metric[s] if metric else s)}}, version,
                          failed=(s == fail_session))


def test_groups_complete_then_sample_oldest_first_and_release():
    rb = ReplayBuffer("sync", n=2)
    _fill(rb, "b", 2, 1)
    _fill(rb, "a", 2, 0)
    rb.add_prompt("c", {}, 1)
    rb.add_trajectory("c", 0, 0, {"response_ids": [1]}, 1)  # only one of two sessions
    assert rb.count(FINISHED) == 2 and rb.inflight() == 1
    meta = rb.sample(2, current_version=1)
    assert meta.keys == ["a_0_0", "a_1_0", "b_0_0", "b_1_0"] and len(rb.q.get_data(meta)) == 4
    assert rb.sample(1, timeout=0.0, pump=lambda: None) is None
    rb.release(meta)
    assert rb.drain_inflight() == 1 and rb.q.size() == 0


def test_dapo_filter_sync_refills_twice_async_once():
    for mode, credit in (("sync", 2), ("colocate_async", 1)):
        asked = []
        rb = ReplayBuffer(mode, n=2, filter_groups_metric="acc", refill_fn=asked.append, max_off_policy_threshold=99)
        _fill(rb, "same", 2, 0, metric=[1.0, 1.0])
        _fill(rb, "diff", 2, 0, metric=[0.0, 1.0])
        assert rb.ready(1) and not rb.ready(2)
        assert asked == [credit]
        assert rb.pop_metrics()["replay_buffer/dapo/evicted_groups"] == 1


def test_staleness_drop_and_wait():
    asked = []
    rb = ReplayBufferAsync(n=1, max_off_policy_threshold=1, max_off_policy_strategy="drop", refill_fn=asked.append)
    _fill(rb, "old", 1, 0)
    _fill(rb, "new", 1, 2)
    meta = rb.sample(1, current_version=2)
    assert meta.keys == ["new_0_0"] and asked == [1]
    m = rb.pop_metrics()
    assert m["replay_buffer/off_policy/evicted_groups"] == 1 and m["replay_buffer/staleness/max"] == 2
    rb = ReplayBufferAsync(n=1, max_off_policy_threshold=1, max_off_policy_strategy="wait")
    rb.add_prompt("p", {}, 0)
    assert rb.may_start_new_prompt(0) and not rb.may_start_new_prompt(1)
    rb.add_trajectory("p", 0, 0, {}, 1)
    assert rb.may_start_new_prompt(1) and rb.sample(1, current_version=5).keys == ["p_0_0"]  # never dropped


def test_failed_group_is_kept_in_sync_mode():
    rb = ReplayBuffer("sync", n=2)
    _fill(rb, "f", 2, 0, fail_session=1)
    assert rb.count(FAILURE) == 1 and rb.ready(1)
