"""Router replay: the experts picked in one pass (recorded per token and layer) drive the routers of a later pass."""
import os
from functools import partial

import torch

os.environ["VERL_ENGINE_DEVICE"] = "cpu"


def _engine():
    from verl_b200.models import get_preset
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead

    eng = NativeEngineWithLMHead(get_preset("tiny-moe"), FSDPEngineConfig(seed=3, micro_batch_size_per_gpu=2), OptimizerConfig(lr=1e-3))
    eng.initialize()
    return eng


def _data():
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(3, 500, (4, 20), generator=g)
    am = torch.ones_like(ids)
    am[2, :4] = 0
    return {"input_ids": ids, "attention_mask": am, "responses": ids[:, -8:], "response_mask": am[:, -8:]}


def test_record_then_replay_reproduces_and_controls_routing():
    from verl_b200.workers.utils.losses import sft_loss

    eng = _engine()
    cfg = eng.arch
    out = eng.infer_batch(dict(_data()) | {"record_routing": True})["model_output"]
    routed = out["routed_experts"]
    assert routed.shape == (4, 20, cfg.num_hidden_layers, cfg.num_experts_per_tok) and routed.dtype == torch.int32
    assert int(routed[2, :4].abs().sum()) == 0                      # padding positions carry nothing
    assert int(routed.max()) < cfg.num_experts
    # the chosen experts of a token are distinct
    r = routed[0, 5, 0].tolist()
    assert len(set(r)) == len(r)
    lp0 = out["log_probs"]
    # same routing replayed: identical outputs
    lp1 = eng.infer_batch(dict(_data()) | {"routed_experts": routed})["model_output"]["log_probs"]
    assert torch.allclose(lp0, lp1, atol=1e-6)
    # different routing imposed: outputs change
    other = (routed + 1) % cfg.num_experts
    lp2 = eng.infer_batch(dict(_data()) | {"routed_experts": other})["model_output"]["log_probs"]
    assert (lp0 - lp2).abs().max() > 1e-4
    # after the router weights moved, replay still follows the recorded experts while a free pass re-routes
    for i in range(cfg.num_hidden_layers):
        w = eng.params.layer(i)["mlp.gate.weight"]
        w.copy_(torch.roll(w, 1, 0))
    rec2 = eng.infer_batch(dict(_data()) | {"record_routing": True})["model_output"]["routed_experts"]
    assert (rec2 != routed).any()
    # training with replay: gradients flow (router weights included) and the step is finite
    res = eng.train_batch(dict(_data()) | {"routed_experts": routed}, partial(sft_loss, None))
    assert torch.isfinite(torch.tensor(res["metrics"]["grad_norm"])) and res["metrics"]["grad_norm"] > 0


def test_grpo_step_with_r2_replay_carries_the_routing_in_the_batch():
    from verl_b200.trainer.main_ppo import main

    t = main(['data.train_batch_size=4', 'data.max_prompt_length=16', 'data.max_response_length=12', 'data.synthetic.num_prompts=16',
              'data.synthetic.prompt_length=16', 'data.synthetic.vocab_high=512', 'actor_rollout_ref.model.path=tiny-moe',
              'actor_rollout_ref.rollout.n=2', 'actor_rollout_ref.actor.ppo_mini_batch_size=4',
              'actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4', 'actor_rollout_ref.actor.use_kl_loss=true',
              'actor_rollout_ref.actor.router_replay.mode=R2', 'actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8',
              'actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=8', 'algorithm.adv_estimator=grpo',
              'reward_model.reward_manager=token_rule', 'trainer.n_gpus_per_node=1', 'trainer.total_epochs=1',
              'trainer.total_training_steps=2', 'trainer.device=cpu', 'trainer.val_before_train=false',
              'actor_rollout_ref.rollout.max_num_seqs=8', 'actor_rollout_ref.rollout.block_size=8', 'trainer.resume_mode=disable',
              'trainer.logger=[]'])
    b = t.last_batch.batch
    assert b["routed_experts"].shape == (8, 28, 2, 2) and b["routed_experts"].dtype == torch.int32


def test_rollout_engine_returns_the_routing_of_every_fed_token():
    """R3: the rollout engine records the experts per token; replaying them in the trainer reproduces the rollout's
    log-probs exactly."""
    from verl_b200.models import FlatParams, get_preset
    from verl_b200.workers.rollout.native.engine import RolloutEngine, SamplingParams

    cfg = get_preset("tiny-moe")
    eng_t = _engine()
    rollout = RolloutEngine(cfg, eng_t.params, max_num_seqs=4, max_model_len=64, block_size=4, eos_token_id=-1, record_routing=True)
    prompts = [[5, 6, 7, 8, 9, 10], [5, 6, 7, 8, 9, 10], [20, 21, 22]]
    outs = rollout.generate(prompts, SamplingParams(temperature=1.0, max_tokens=6))
    L, k = cfg.num_hidden_layers, cfg.num_experts_per_tok
    for o in outs:
        re_ = o.extra_fields["routed_experts"]
        assert re_.shape == (len(o.prompt_ids) + len(o.token_ids) - 1, L, k) and int(re_.max()) < cfg.num_experts
    assert torch.equal(outs[0].extra_fields["routed_experts"][:6], outs[1].extra_fields["routed_experts"][:6])  # shared prompt
    # trainer forward over prompt + response with the recorded routing == rollout log-probs
    P_len, R = 6, 6
    ids = torch.zeros(3, P_len + R, dtype=torch.long)
    am = torch.zeros_like(ids)
    routed = torch.zeros(3, P_len + R, L, k, dtype=torch.int32)
    for i, o in enumerate(outs):
        p = len(o.prompt_ids)
        ids[i, P_len - p : P_len] = torch.tensor(o.prompt_ids)
        ids[i, P_len:] = torch.tensor(o.token_ids)
        am[i, P_len - p :] = 1
        re_ = o.extra_fields["routed_experts"].int()
        routed[i, P_len - p : P_len - p + re_.shape[0]] = re_
    data = {"input_ids": ids, "attention_mask": am, "responses": ids[:, P_len:], "routed_experts": routed}
    lp = eng_t.infer_batch(data)["model_output"]["log_probs"]
    roll_lp = torch.tensor([o.log_probs for o in outs])
    assert torch.allclose(lp, roll_lp, atol=1e-4)


def test_grpo_step_with_r3_replay_uses_the_rollout_routing():
    from verl_b200.trainer.main_ppo import main

    t = main(['data.train_batch_size=4', 'data.max_prompt_length=16', 'data.max_response_length=12', 'data.synthetic.num_prompts=16',
              'data.synthetic.prompt_length=16', 'data.synthetic.vocab_high=512', 'actor_rollout_ref.model.path=tiny-moe',
              'actor_rollout_ref.rollout.n=2', 'actor_rollout_ref.actor.ppo_mini_batch_size=4',
              'actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4', 'actor_rollout_ref.actor.use_kl_loss=true',
              'actor_rollout_ref.actor.router_replay.mode=R3', 'actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8',
              'actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=8', 'algorithm.adv_estimator=grpo',
              'reward_model.reward_manager=token_rule', 'trainer.n_gpus_per_node=1', 'trainer.total_epochs=1',
              'trainer.total_training_steps=2', 'trainer.device=cpu', 'trainer.val_before_train=false',
              'actor_rollout_ref.rollout.max_num_seqs=8', 'actor_rollout_ref.rollout.block_size=8', 'trainer.resume_mode=disable',
              'trainer.logger=[]'])
    b = t.last_batch.batch
    assert b["routed_experts"].shape == (8, 28, 2, 2)
    m = b["response_mask"].bool()
    # with the rollout's routing replayed, the recomputed behaviour log-probs equal the rollout's
    assert (torch.exp(b["old_log_probs"]) - torch.exp(b["rollout_log_probs"])).abs()[m].max() < 1e-4
