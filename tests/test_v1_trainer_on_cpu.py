"""v1 trainers end to end on CPU with the tiny model: sync and colocate_async both train for two steps."""
import os

import pytest

ARGS = ['data.train_batch_size=4', 'data.max_prompt_length=16', 'data.max_response_length=12', 'data.synthetic.num_prompts=32',
        'data.synthetic.prompt_length=16', 'data.synthetic.vocab_high=512', 'actor_rollout_ref.model.path=tiny-qwen2',
        'actor_rollout_ref.rollout.n=2', 'actor_rollout_ref.actor.ppo_mini_batch_size=4',
        'actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8', 'actor_rollout_ref.actor.use_kl_loss=true',
        'actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=16', 'actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=16',
        'algorithm.adv_estimator=grpo', 'reward_model.reward_manager=token_rule', 'trainer.n_gpus_per_node=1', 'trainer.total_epochs=4',
        'trainer.total_training_steps=2', 'trainer.device=cpu', 'trainer.val_before_train=false', 'actor_rollout_ref.rollout.max_num_seqs=16',
        'actor_rollout_ref.rollout.block_size=8', 'trainer.resume_mode=disable', 'trainer.use_v1=true', 'trainer.worker_group=inprocess']


@pytest.mark.parametrize("mode", ["sync", "colocate_async"])
def test_v1_modes_train(mode, monkeypatch):
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    from verl_b200.trainer.main_ppo import main

    t = main(ARGS + [f"trainer.v1.trainer_mode={mode}"])
    assert type(t).trainer_mode == mode
    assert t.global_steps == 3 and t.param_version == 2
    assert t.last_batch.batch["advantages"].shape == (8, 12)
    if mode == "colocate_async":
        # the warm-up batch was generated under older weights and is still usable (threshold 1)
        assert t.replay_buffer.inflight() + t.replay_buffer.count("finished") > 0


def test_separate_async_single_pool_and_switch_controller(monkeypatch):
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    from verl_b200.trainer.main_ppo import main
    from verl_b200.trainer.ppo.v1.trainer_separate_async import SwitchController

    t = main(ARGS + ["trainer.v1.trainer_mode=separate_async", "trainer.v1.parameter_sync_step=2", "trainer.total_training_steps=1"])
    assert t.param_version == 1 and t.topo.R == 0  # two optimizer rounds, one weight hand-over
    sc = SwitchController(enabled=True, ratio=2.0)
    assert sc.should_switch(0.0)  # no cost measured yet: switching is free
    sc.record_switch_cost(1.0)
    assert not sc.should_switch(1.0) and sc.should_switch(2.5)
    sc.record_wait(3.0)
    assert not sc.should_switch(2.5)  # on average only 0.5 s of waiting is left: below 2 x cost
    assert not SwitchController(enabled=False).should_switch(100.0)


def _split_proc(rank, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      VERL_ENGINE_DEVICE="cpu")
    try:
        from verl_b200.trainer.main_ppo import main

        args = [a for a in ARGS if not a.startswith("trainer.worker_group")] + [
            "trainer.worker_group=spmd", "trainer.v1.trainer_mode=separate_async", "trainer.v1.rollout_ranks=1",
            "trainer.v1.hybrid_switch=false", "trainer.total_training_steps=2"]
        res = main(args)
        if isinstance(res, dict):
            q.put((rank, res))
        else:
            q.put((rank, {"param_version": res.param_version, "steps": res.global_steps}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_separate_async_two_processes_trainer_and_rollout_rank():
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_split_proc, args=(r, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=240) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    assert "error" not in res[0], res[0]["error"]
    assert "error" not in res[1], res[1]["error"]
    assert res[0]["param_version"] == 2 and res[0]["steps"] == 3
    assert res[1]["groups"] >= 8 and res[1]["weight_syncs"] >= 1  # all samples came from the rollout rank


def test_one_step_off_single_pool(monkeypatch):
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    from verl_b200.experimental.one_step_off_policy.main_ppo import main

    t = main(ARGS + ["trainer.total_training_steps=3"])
    assert type(t).__name__ == "OneStepOffRayTrainer" and t.param_version == 3
    ages = t.last_batch  # batches after the first were generated one version earlier
    assert ages is not None


def test_async_trainer_checkpoints_its_buffer_and_reissues_inflight_prompts(monkeypatch, tmp_path):
    """The asynchronous trainers keep the replay buffer in the checkpoint; after a resume the groups that were still being
    generated start again from their stored prompts (partial trajectories dropped), finished groups are trained on as
    they are, and training goes on."""
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    from verl_b200.trainer.main_ppo import main

    base = [a for a in ARGS if not a.startswith(("trainer.resume_mode", "trainer.total_training_steps"))] + [
        "trainer.v1.trainer_mode=colocate_async", f"trainer.default_local_dir={tmp_path}", "trainer.save_freq=2"]
    t = main(base + ["trainer.resume_mode=disable", "trainer.total_training_steps=2"])
    state = tmp_path / "global_step_2" / "transfer_queue" / "state.pt"
    assert state.exists()
    import torch

    saved = torch.load(state, weights_only=False)
    tags = saved["tags"]["train"]
    live = [k for k, v in tags.items() if v.get("kind") == "prompt" and v.get("status") in ("pending", "running")]
    done = [k for k, v in tags.items() if v.get("kind") == "prompt" and v.get("status") == "finished"]
    assert saved["metadata"] == {"global_steps": 2, "param_version": 2} and (live or done)

    t2 = main(base + ["trainer.resume_mode=auto", "trainer.total_training_steps=3"])
    assert t2.global_steps == 4 and t2.param_version == 3            # resumed at step 2, trained step 3
    q = t2.replay_buffer.q
    for uid in live:                                                 # re-issued groups: consumed, or complete again, never half
        if uid in q.list_keys("train"):
            tg = q.get_tags(uid, "train")
            assert tg["done"] <= tg["n"] and tg["start_version"] >= 2


def test_fit_step_runs_the_overridable_phases_in_order(monkeypatch):
    """``fit_step`` is a template over ``_fit_*`` phases (the names of ``verl/experimental/separation/ray_trainer.py``):
    wrapping each phase records the order, and overriding one changes only that part of the step."""
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    from verl_b200.trainer.main_ppo import main

    args = [a for a in ARGS if not a.startswith(("trainer.use_v1", "trainer.total_training_steps"))]
    t = main(args + ["trainer.use_v1=false", "trainer.total_training_steps=1"])
    assert t.global_steps == 2
    order = []
    names = ["_fit_prepare_step", "_fit_start_profile", "_fit_get_batch", "_fit_generate", "_fit_balance", "_fit_compute_reward",
             "_fit_compute_log_prob", "_fit_compute_ref_log_prob", "_fit_compute_critic", "_fit_compute_teacher_logprobs",
             "_fit_compute_advantage",
             "_fit_update_critic", "_fit_update_actor", "_fit_update_weights", "_fit_dump_data", "_fit_validate",
             "_fit_save_checkpoint", "_fit_stop_profile", "_fit_collect_metrics", "_fit_experimental", "_fit_postprocess_step"]
    for n in names:
        def wrap(*a, _n=n, _f=getattr(t, n), **k):
            order.append(_n)
            return _f(*a, **k)
        monkeypatch.setattr(t, n, wrap)

    def doubled_reward(batch, _f=t._fit_compute_reward):
        batch = _f(batch)
        batch.batch["token_level_scores"] = batch.batch["token_level_scores"] * 2
        return batch

    monkeypatch.setattr(t, "_fit_compute_reward", doubled_reward)
    t.total_training_steps = 5
    metrics, timing = t.fit_step(next(iter(t.train_dataloader)))
    assert order == names and t.global_steps == 3 and metrics["training/global_step"] == 2
    assert {"gen", "old_log_prob", "ref", "adv", "update_actor", "update_weights", "step"} <= set(timing)
    scores = t.last_batch.batch["token_level_scores"].sum(-1)
    assert abs(metrics["critic/score/mean"] - scores.mean().item()) < 1e-5 and "actor/entropy" in metrics
    # the coarse phases used by the benchmark and the asynchronous trainers are the same methods, grouped
    order.clear()
    t.train_step(next(iter(t.train_dataloader)))
    assert order == names[2:15] + ["_fit_collect_metrics"]


def test_critic_token_budget_reaches_value_inference(monkeypatch):
    """``critic.use_dynamic_bsz`` with ``forward_max_token_len_per_gpu`` splits ``compute_values`` into micro-batches under
    the token budget (one micro-batch of the whole batch does not fit a GPU at the benchmark's size)."""
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    from verl_b200.trainer.main_ppo import main

    args = [a for a in ARGS if not a.startswith(("trainer.use_v1", "trainer.total_training_steps", "algorithm.adv_estimator",
                                                  "actor_rollout_ref.actor.use_kl_loss"))]
    t = main(args + ["trainer.use_v1=false", "trainer.total_training_steps=1", "algorithm.adv_estimator=gae",
                     "actor_rollout_ref.actor.use_kl_loss=false", "critic.model.path=tiny-qwen2", "critic.ppo_mini_batch_size=4",
                     "critic.use_dynamic_bsz=true", "critic.ppo_max_token_len_per_gpu=64", "critic.forward_max_token_len_per_gpu=56"])
    eng = t.critic_wg._workers[0].engine
    ec = eng.engine_config
    assert ec.use_dynamic_bsz and ec.max_token_len_per_gpu == 64 and ec.infer_max_token_len_per_gpu == 56
    data = {k: t.last_batch.batch[k] for k in ("input_ids", "attention_mask", "position_ids", "responses", "response_mask")}
    parts = eng._micro_batches(dict(data), forward_only=True)
    lens = [int(p["attention_mask"].sum()) for p in parts]
    assert len(parts) >= 2 and sum(lens) == int(data["attention_mask"].sum()), lens
    assert all(n <= 56 or p["input_ids"].shape[0] == 1 for n, p in zip(lens, parts)), lens
    assert "critic/vf_loss" in t.metrics and t.last_batch.batch["values"].shape == (8, 12)


def test_group_relative_advantage_over_sessions_with_several_rows():
    """Only the final row of a session takes part in the group statistics; the other rows of the session get its value on
    their own response tokens. Token-wise estimators see the batch unchanged."""
    import numpy as np
    import torch

    from verl_b200 import DataProto
    from verl_b200.trainer.ppo.v1.utils import (compute_advantage_for_multi_trajectories, has_multi_trajectory_sessions,
                                                 split_trajectory_key)

    assert split_trajectory_key("a_b_c_3_1") == ("a_b_c", "3", 1)
    keys = ["p_0_0", "p_0_1", "p_1_0", "q_0_0", "q_1_0", "q_1_1"]
    assert has_multi_trajectory_sessions(keys) and not has_multi_trajectory_sessions(["p_0_0", "p_1_0"])
    R = 4
    mask = torch.tensor([[1, 1, 0, 0], [1, 1, 1, 0], [1, 1, 1, 1], [0, 1, 1, 0], [1, 0, 0, 0], [1, 1, 0, 0]], dtype=torch.float32)
    # outcome scores sit on the final rows: sessions p/0 -> 1.0, p/1 -> 0.0, q/0 -> 0.5, q/1 -> 2.5; the score on the
    # non-final rows (p_0_0, q_1_0) must not matter
    score = torch.zeros(6, R)
    score[1, 2], score[2, 3], score[3, 2], score[5, 1] = 1.0, 0.0, 0.5, 2.5
    score[0, 1], score[4, 0] = 9.0, -9.0
    data = DataProto.from_dict(tensors={"token_level_rewards": score, "response_mask": mask, "responses": torch.zeros(6, R, dtype=torch.int64)},
                               non_tensors={"uid": np.array(["p", "p", "p", "q", "q", "q"], dtype=object)})
    out = compute_advantage_for_multi_trajectories(data, keys, "grpo", num_repeat=2, norm_adv_by_std_in_grpo=True)
    adv = out.batch["advantages"]
    # group p: scores (1, 0): mean 0.5, unbiased std 0.7071 -> +-0.7071; group q: (0.5, 2.5): mean 1.5, std 1.4142 -> -+0.7071
    a = 0.5 / (0.5 ** 0.5 + 1e-6)
    want = torch.tensor([a, a, -a, -a, a, a]).unsqueeze(-1) * mask
    assert torch.allclose(adv, want, atol=1e-4), adv
    assert torch.equal(out.batch["returns"], adv)
    # a token-wise estimator is passed through
    data2 = DataProto.from_dict(tensors={"token_level_rewards": score.clone(), "response_mask": mask, "values": torch.zeros(6, R),
                                         "responses": torch.zeros(6, R, dtype=torch.int64)},
                                non_tensors={"uid": np.array(["p", "p", "p", "q", "q", "q"], dtype=object)})
    out2 = compute_advantage_for_multi_trajectories(data2, keys, "gae", gamma=1.0, lam=1.0)
    assert out2.batch["advantages"].shape == (6, R) and float(out2.batch["advantages"][0].abs().sum()) > 0   # row 0's own reward counted


def test_sessions_that_return_several_rows_train_through_the_replay_buffer(monkeypatch):
    """An agent loop that cuts its session into two rows: both are stored (index 0 and 1), the group completes on the last
    one, and the trainer's batch holds every row with its session's advantage."""
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    import copy

    from verl_b200.experimental.agent_loop import register
    from verl_b200.experimental.agent_loop.single_turn_agent_loop import SingleTurnAgentLoop
    from verl_b200.trainer.main_ppo import main

    @register("two_piece_agent")
    class TwoPieces(SingleTurnAgentLoop):
        async def run(self, sampling_params, **kwargs):
            whole = await super().run(sampling_params, **kwargs)
            cut = max(1, len(whole.response_ids) // 2)
            first = copy.copy(whole)
            first.response_ids, first.response_mask = whole.response_ids[:cut], whole.response_mask[:cut]
            first.response_logprobs = None if whole.response_logprobs is None else whole.response_logprobs[:cut]
            first.reward_score = None
            second = copy.copy(whole)
            second.prompt_ids = whole.prompt_ids + whole.response_ids[:cut]
            second.response_ids, second.response_mask = whole.response_ids[cut:], whole.response_mask[cut:]
            second.response_logprobs = None if whole.response_logprobs is None else whole.response_logprobs[cut:]
            return [first, second] if second.response_ids else [first]

    t = main(ARGS + ["trainer.v1.trainer_mode=sync", "trainer.total_training_steps=1", "data.max_prompt_length=32",
                     "+actor_rollout_ref.rollout.agent.default_agent_loop=two_piece_agent"])
    b = t.last_batch
    keys = b.non_tensor_batch["__traj_key__"].tolist()
    assert len(keys) == 16 and sorted({k.rsplit("_", 1)[1] for k in keys}) == ["0", "1"]     # 4 prompts x 2 sessions x 2 rows
    adv, m = b.batch["advantages"], b.batch["response_mask"].bool()
    by_session = {}
    for i, k in enumerate(keys):
        v = adv[i][m[i]]
        assert v.numel() > 0 and bool((v == v[0]).all())
        by_session.setdefault(k.rsplit("_", 1)[0], []).append(float(v[0]))
    assert all(len(v) == 2 and abs(v[0] - v[1]) < 1e-6 for v in by_session.values())          # both rows share the session's value
    assert t.global_steps == 2 and "actor/pg_loss" in t.metrics


def test_rounds_of_one_step_are_reduced_by_name():
    import torch

    from verl_b200.trainer.ppo.v1.utils import StepMetricsAggregator as A

    assert A.rule("actor/lr") == "last" and A.rule("timing_s/gen") == "sum" and A.rule("timing_per_token_ms/adv") == "sum"
    assert A.rule("training/off_policy/evicted_samples") == "sum" and A.rule("response_length/max") == "max"
    assert A.rule("critic/score/mean") == "weighted" and A.rule("actor/pg_loss") == "weighted" and A.rule("training/global_step") == "last"
    a = A()
    assert a.get_aggregated_metrics() == {}
    a.add_step_metrics({"actor/pg_loss": 1.0, "actor/lr": 1e-3, "timing_s/gen": 2.0, "response_length/max": 10, "response_length/min": 3,
                        "global_seqlen/max": 90, "global_seqlen/min": 30, "global_seqlen/minmax_diff": 60,
                        "training/off_policy/evicted_samples": 2, "training/off_policy/evicted_samples_staleness/mean": 3.0,
                        "hist": {"0.0": 2, "1.0": 1}, "flag": True, "t": torch.tensor(4.0)}, sample_count=8)
    a.add_step_metrics({"actor/pg_loss": 4.0, "actor/lr": 5e-4, "timing_s/gen": 3.0, "response_length/max": 7, "response_length/min": 1,
                        "global_seqlen/max": 80, "global_seqlen/min": 20, "global_seqlen/minmax_diff": 60,
                        "training/off_policy/evicted_samples": 6, "training/off_policy/evicted_samples_staleness/mean": 5.0,
                        "hist": {"1.0": 4}, "t": torch.tensor(8.0)}, sample_count=24)
    out = a.get_aggregated_metrics()
    assert out["actor/pg_loss"] == pytest.approx((1.0 * 8 + 4.0 * 24) / 32) and out["actor/lr"] == 5e-4 and out["timing_s/gen"] == 5.0
    assert out["response_length/max"] == 10 and out["response_length/min"] == 1 and out["global_seqlen/minmax_diff"] == 70
    assert out["training/off_policy/evicted_samples"] == 8
    assert out["training/off_policy/evicted_samples_staleness/mean"] == pytest.approx((3.0 * 2 + 5.0 * 6) / 8)   # weighted by evictions
    assert out["hist"] == {"0.0": 2, "1.0": 5} and "flag" not in out and out["t"] == pytest.approx((4 * 8 + 8 * 24) / 32)


def test_adaptive_switch_threshold_and_benefit_rule():
    from verl_b200.trainer.config.config import BaseModelConfig, HybridRolloutSwitchConfig, ModuleConfig, ProfileConfig
    from verl_b200.trainer.ppo.v1.hybrid_switch import AdaptiveSwitchThreshold, SwitchCostWindow, switch_is_worth_it

    with pytest.raises(ValueError):
        HybridRolloutSwitchConfig(switch_threshold_ratio=0.0)
    with pytest.raises(ValueError):
        HybridRolloutSwitchConfig(switch_cost_window_size=0)
    assert ProfileConfig().step_start == -1 and ModuleConfig().path is None and BaseModelConfig().lora == {}
    cfg = HybridRolloutSwitchConfig(enable_switch=True, switch_threshold_ratio=0.4, switch_threshold_step_up=0.05,
                                    switch_threshold_step_down=0.03, switch_threshold_release_steps=2)
    t = AdaptiveSwitchThreshold(cfg, train_batch_size=64, parameter_sync_step=4)
    assert t.threshold() == 26                       # round(0.4 * 64), above one mini-batch of 16
    assert t.adapt(True) == pytest.approx(0.4)       # one idle step: not yet
    assert t.adapt(True) == pytest.approx(0.45)      # two in a row: up
    assert t.adapt(True) == pytest.approx(0.50) and t.threshold() == 32
    assert t.adapt(False) == pytest.approx(0.50)     # one calm step resets the idle count, no move yet
    assert t.adapt(True) == pytest.approx(0.50)      # ... and an idle step resets the calm count
    assert t.adapt(False) == pytest.approx(0.50) and t.adapt(False) == pytest.approx(0.47)
    for _ in range(40):
        t.adapt(False)
    assert t.ratio == pytest.approx(0.25) and t.threshold() == 16     # floor: one round's share of the batch
    for _ in range(40):
        t.adapt(True)
    assert t.ratio == 1.0 and t.threshold() == 64
    fixed = AdaptiveSwitchThreshold(HybridRolloutSwitchConfig(adaptive_switch_threshold=False), 64)
    assert fixed.adapt(True) == fixed.adapt(True) == 0.4
    w = SwitchCostWindow(size=2)
    assert w.effective_cost() is None
    for c in (4.0, 2.0, 1.0):
        w.to_rollout.append(c)
    w.to_trainer.append(3.0)
    assert w.effective_cost() == pytest.approx(1.5 + 3.0)            # the window keeps the last two
    assert not switch_is_worth_it(0, 1.0, 2.0, 1.0)
    assert switch_is_worth_it(10, None, 2.0, 1.0) and switch_is_worth_it(10, 1.0, 2.0, None)
    assert switch_is_worth_it(10, 1.0, 2.0, 4.9) and not switch_is_worth_it(10, 1.0, 2.0, 5.1)     # saves 10 * 1 * (1 - 1/2) = 5 s
