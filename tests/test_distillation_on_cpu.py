"""Distillation: forward-KL top-k loss against a dense reference, hidden-state path, teacher batching and routing."""
import pytest
import asyncio

import torch

from verl_b200.experimental.teacher_loop import AsyncTeacherLLMServerManager, MultiTeacherModelManager, TeacherModelManager
from verl_b200.models import DecoderModel, FlatParams, PackedBatch, get_preset
from verl_b200.trainer.distillation.losses import (DistillationConfig, DistillationLossConfig, compute_forward_kl_topk,
                                                   distillation_loss, student_topk_log_probs)


def test_forward_kl_topk_matches_dense_kl_when_k_is_vocab():
    torch.manual_seed(0)
    s, t = torch.randn(2, 5, 11), torch.randn(2, 5, 11)
    lp_t = torch.log_softmax(t, -1)
    ids = torch.arange(11).expand(2, 5, 11)
    cfg = DistillationLossConfig(log_prob_min_clamp=None)
    out = compute_forward_kl_topk(s, lp_t, ids, cfg)
    dense = torch.nn.functional.kl_div(torch.log_softmax(s, -1), lp_t, log_target=True, reduction="none").sum(-1)
    assert torch.allclose(out["distillation_losses"], dense, atol=1e-5)
    assert torch.allclose(out["teacher_mass"], torch.ones(2, 5), atol=1e-5)
    v, i = torch.topk(lp_t, 3, -1)  # k < V with the tail term: still non-negative and below the dense KL + tail
    out3 = compute_forward_kl_topk(s, v, i, DistillationLossConfig(log_prob_min_clamp=None, use_tail_term=True))
    assert (out3["distillation_losses"] > -1e-6).all() and (out3["distillation_losses"] <= dense + 1e-5).all()


def test_hidden_path_and_scalar_loss_backward():
    torch.manual_seed(0)
    h = torch.randn(7, 16, requires_grad=True)
    W = torch.randn(32, 16, requires_grad=True)
    ids = torch.randint(0, 32, (7, 4))
    lq = student_topk_log_probs(h, W, ids, chunk=3)
    ref = torch.log_softmax(h @ W.t(), -1).gather(-1, ids)
    assert torch.allclose(lq, ref, atol=1e-5)
    lp_t = torch.log_softmax(torch.randn(7, 4), -1)
    data = {"teacher_logprobs": lp_t.view(1, 7, 4), "teacher_ids": ids.view(1, 7, 4), "response_mask": torch.ones(1, 7)}
    dc = DistillationConfig(enabled=True, distillation_loss=DistillationLossConfig(loss_mode="forward_kl_topk"))
    loss, m = distillation_loss({"loss_agg_mode": "token-mean"}, dc, {"topk_log_probs": lq.view(1, 7, 4)}, data)
    loss.backward()
    assert h.grad.abs().sum() > 0 and "distillation/loss_max" in m and "distillation/student_mass" in m
    dc2 = DistillationConfig(enabled=True, distillation_loss=DistillationLossConfig(loss_mode="k3"))
    lp = torch.randn(1, 7).clamp(-3, 0).requires_grad_()
    loss2, _ = distillation_loss({"loss_agg_mode": "token-mean"}, dc2, {"log_probs": lp}, {"teacher_logprobs": lp.detach() - 0.1, "response_mask": torch.ones(1, 7)})
    assert loss2.item() > 0


def test_teacher_servers_batch_requests_and_route_by_key():
    cfg = get_preset("tiny-qwen2")
    models = []
    for seed in (1, 2):
        P = FlatParams(cfg, dtype=torch.float32)
        P.init_weights(seed=seed, std=0.1)
        models.append(DecoderModel(cfg, P))
    a = TeacherModelManager.from_models("math", [models[0]], topk=4)
    b = TeacherModelManager.from_models("code", [models[1]], topk=4)
    mgr = AsyncTeacherLLMServerManager(MultiTeacherModelManager({"math": a, "code": b}), response_length=6)

    async def go():
        return await asyncio.gather(*[mgr.compute_teacher_logprobs(f"r{i}", [5, 6, 7], [8, 9, 10, 11], key)
                                      for i, key in enumerate(["math", "math", "code", "unknown"])])

    outs = asyncio.run(go())
    assert outs[0]["teacher_ids"].shape == (6, 4) and (outs[0]["teacher_logprobs"][4:] == 0).all()
    assert torch.equal(outs[0]["teacher_ids"], outs[1]["teacher_ids"]) and torch.equal(outs[0]["teacher_ids"], outs[3]["teacher_ids"])
    assert not torch.equal(outs[0]["teacher_logprobs"], outs[2]["teacher_logprobs"])
    assert list(a.servers.values())[0].num_forwards == 1  # three concurrent requests shared one forward
    # the record agrees with a dense forward of the teacher
    lg = models[0].forward_logits(PackedBatch.from_lengths(torch.tensor([5, 6, 7, 8, 9, 10, 11]), [7])).float()
    v, i = torch.topk(torch.log_softmax(lg, -1)[2:6], 4, -1)
    assert torch.equal(outs[0]["teacher_ids"][:4], i) and torch.allclose(outs[0]["teacher_logprobs"][:4], v, atol=1e-5)


def test_agent_loop_attaches_teacher_records_to_sampled_trajectories_only():
    """With a teacher manager the agent-loop worker asks the teacher picked by the sample's routing field for top-k
    log-probs of every sampled trajectory and batches them as [b, R, k]; validation batches carry none."""
    from verl_b200 import DataProto
    from verl_b200.experimental.agent_loop import AgentLoopManager
    from verl_b200.utils.config import DictConfig
    from verl_b200.workers.rollout.llm_server import LLMServerManager
    from verl_b200.workers.rollout.native.engine import RolloutEngine
    import numpy as np

    cfg = get_preset("tiny-qwen2")
    teachers = {}
    for name, seed in (("math", 1), ("code", 2)):
        P = FlatParams(cfg, dtype=torch.float32)
        P.init_weights(seed=seed, std=0.1)
        teachers[name] = TeacherModelManager.from_models(name, [DecoderModel(cfg, P)], topk=4)
    tm = AsyncTeacherLLMServerManager(MultiTeacherModelManager(teachers), response_length=6)
    config = DictConfig({"distillation": {"enabled": True, "teacher_key": "domain"},
                         "actor_rollout_ref": {"rollout": {"name": "native", "prompt_length": 8, "response_length": 6, "temperature": 1.0,
                                                           "top_p": 1.0, "top_k": -1, "do_sample": True, "calculate_log_probs": True,
                                                           "tensor_model_parallel_size": 1, "agent": {"num_workers": 1},
                                                           "val_kwargs": {"temperature": 0.0, "do_sample": False}}}})
    S = FlatParams(cfg, dtype=torch.float32)
    S.init_weights(seed=3, std=0.1)
    eng = RolloutEngine(cfg, S, max_num_seqs=4, max_model_len=64, block_size=8, sync_interval=2, eos_token_id=-1)

    async def go(validate):
        mgr = await LLMServerManager.create(config.actor_rollout_ref.rollout, engines=[eng], model_config=None)
        alm = AgentLoopManager(config, mgr, teacher_server_manager=tm)
        ids = torch.randint(3, 500, (4, 8))
        batch = DataProto.from_dict(tensors={"input_ids": ids, "attention_mask": torch.ones(4, 8, dtype=torch.int64)},
                                    non_tensors={"domain": np.array(["math", "code", "math", "other"], dtype=object)},
                                    meta_info={"temperature": 1.0, "validate": validate})
        return await alm.generate_sequences_async(batch)

    out = asyncio.run(go(False))
    ti, tl = out.batch["teacher_ids"], out.batch["teacher_logprobs"]
    assert ti.shape == (4, 6, 4) and tl.shape == (4, 6, 4) and (tl <= 0).all()
    assert "teacher_ids" not in out.non_tensor_batch
    # row 1 was scored by the other teacher: re-scoring its tokens with each teacher tells which one answered
    seq = out.batch["input_ids"][1].tolist()
    for name, same in (("code", True), ("math", False)):
        ref = asyncio.run(AsyncTeacherLLMServerManager(MultiTeacherModelManager(teachers), 6).compute_teacher_logprobs("x", seq[:8], seq[8:], name))
        assert torch.allclose(ref["teacher_logprobs"], tl[1], atol=1e-5) == same
    assert "teacher_ids" not in asyncio.run(go(True)).batch.keys()


def test_on_policy_distillation_end_to_end_through_the_trainer(monkeypatch):
    """``distillation.enabled`` builds the teacher, scores every trajectory with the sampled token's teacher log-prob and
    trains the actor on task loss + k3 term; with ``use_task_rewards=false`` the distillation term alone drives the update."""
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    from tests.test_v1_trainer_on_cpu import ARGS
    from verl_b200.trainer.main_ppo import main

    args = [a for a in ARGS if not a.startswith(("trainer.use_v1", "trainer.total_training_steps"))] + [
        "trainer.use_v1=false", "trainer.total_training_steps=1", "distillation.enabled=true",
        "distillation.teacher_models.teacher_model.model_path=tiny-qwen2"]
    t = main(args)
    b = t.last_batch.batch
    assert b["teacher_logprobs"].shape == (8, 12, 1) and b["teacher_ids"].shape == (8, 12, 1)
    m = b["response_mask"].bool()
    assert torch.equal(b["teacher_ids"][..., 0][m], b["responses"][m])          # the record is about the sampled tokens
    assert (b["teacher_logprobs"][..., 0][m] < 0).all() and (b["teacher_logprobs"][..., 0][~m] == 0).all()
    assert t.metrics["actor/distillation/loss"] > 0 and "actor/pg_loss" in t.metrics and "timing_s/teacher" in t.metrics
    t2 = main(args + ["distillation.distillation_loss.use_task_rewards=false"])
    assert t2.metrics["actor/distillation/loss"] > 0 and "actor/pg_loss" not in t2.metrics and t2.metrics["actor/grad_norm"] > 0
    with pytest.raises(NotImplementedError, match="forward_kl_topk"):
        main(args + ["distillation.distillation_loss.loss_mode=forward_kl_topk"])
