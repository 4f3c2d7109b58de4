"""Prime reward manager, prefix-grouper utilities, vocabulary-parallel distillation KL, separation tables."""
import os
import socket

import numpy as np
import torch

os.environ["VERL_ENGINE_DEVICE"] = "cpu"


def _score(data_source, solution_str, ground_truth, extra_info=None):
    if "sleep" in solution_str:
        import time

        time.sleep(30)
    if "boom" in solution_str:
        raise RuntimeError("scorer failed")
    return 1.0 if solution_str.strip() == str(ground_truth) else 0.0


class _Tok:
    def decode(self, ids, skip_special_tokens=True):
        return {1: "7", 2: "sleep", 3: "boom", 4: "9"}[int(ids[0])]


def test_prime_reward_manager_scores_in_parallel_with_time_limit():
    from verl_b200.protocol import DataProto
    from verl_b200.workers.reward_manager import get_reward_manager_cls

    resp = torch.tensor([[1, 0], [2, 0], [3, 0], [4, 4]])
    am = torch.tensor([[1, 1, 1, 0], [1, 1, 1, 0], [1, 1, 1, 0], [1, 1, 1, 1]])
    data = DataProto.from_dict(tensors={"responses": resp, "attention_mask": am, "prompts": torch.ones(4, 2, dtype=torch.long)},
                               non_tensors={"reward_model": np.array([{"ground_truth": "7"}] * 4, dtype=object),
                                            "data_source": np.array(["t"] * 4, dtype=object)})
    rm = get_reward_manager_cls("prime")(_Tok(), compute_score=_score, num_processes=4, timeout=1.5)
    out = rm(data, return_dict=True)
    r = out["reward_tensor"]
    assert r[0].tolist() == [1.0, 0.0]            # correct answer, reward on the last valid token
    assert r[1].sum() == 0 and r[2].sum() == 0    # timed out / raised -> 0
    assert r[3].tolist() == [0.0, 0.0] and out["reward_extra_info"]["acc"] == [1.0, 0.0, 0.0, 0.0]


def test_prefix_grouper_utils_structure_and_forward():
    from verl_b200.models import get_preset
    from verl_b200.trainer.ppo.prefix_grouper_utils import (build_pg_from_micro_batch, build_position_ids_for_prefix_grouper,
                                                            forward_micro_batch_with_prefix_grouper, shared_prefix_token_savings)
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead

    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(3, 500, (2, 6), generator=g)
    ids = torch.cat([prompt.repeat_interleave(2, 0), torch.randint(3, 500, (4, 5), generator=g)], 1)
    am = torch.ones_like(ids)
    am[2:, :2] = 0                                 # second group's prompt is left-padded
    am[1, -2:] = 0
    mb = {"input_ids": ids, "attention_mask": am, "responses": ids[:, -5:]}
    pg = build_pg_from_micro_batch(mb)
    assert [g_["rows"] for g_ in pg["groups"]] == [[0, 1], [2, 3]] and pg["groups"][1]["prefix_len"] == 4
    assert pg["groups"][0]["suffix_lens"] == [5, 3]
    pos = build_position_ids_for_prefix_grouper(pg)
    assert pos[:6].tolist() == list(range(6)) and pos[6:11].tolist() == list(range(6, 11)) and pos[11:14].tolist() == [6, 7, 8]
    shared, plain = shared_prefix_token_savings(pg)
    assert plain - shared == 6 + 4
    eng = NativeEngineWithLMHead(get_preset("tiny-llama"), FSDPEngineConfig(seed=1), OptimizerConfig(lr=1e-3))
    eng.initialize()
    out = forward_micro_batch_with_prefix_grouper(eng, mb)
    ref = eng.infer_batch(dict(mb) | {"response_mask": am[:, -5:]})["model_output"]["log_probs"]
    assert torch.allclose(out["log_probs"], ref, atol=1e-5)


def _vp_proc(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        import torch.distributed as dist

        from verl_b200.ops import functional as F
        from verl_b200.trainer.distillation.vocab_parallel import compute_forward_kl_topk_vocab_parallel

        dist.init_process_group("gloo", rank=rank, world_size=world)
        g = torch.Generator().manual_seed(0)
        T, V, H, k = 6, 32, 16, 4
        h = torch.randn(T, H, generator=g)
        w = torch.randn(V, H, generator=g) * 0.3
        labels = torch.randint(0, V, (T,), generator=g)
        t_ids = torch.stack([torch.randperm(V, generator=g)[:k] for _ in range(T)])
        t_lp = torch.log_softmax(torch.randn(T, k, generator=g), -1) - 0.1
        Vl = V // world
        # fused head on vocabulary slices
        lp, ent, lse = F.lmhead_logprob_entropy_vocab_parallel(h, w[rank * Vl:(rank + 1) * Vl], labels, 1.0, rank * Vl, dist.group.WORLD)
        lp_r, ent_r, lse_r = F.lmhead_logprob_entropy(h, w, labels, 1.0)
        ok_head = torch.allclose(lp, lp_r, atol=1e-5) and torch.allclose(ent, ent_r, atol=1e-5) and torch.allclose(lse, lse_r, atol=1e-5)
        # backward of the slice with global statistics: partial d_hidden sums to the full one
        g_lp, g_ent = torch.randn(T, generator=g), torch.randn(T, generator=g)
        dw = torch.zeros(Vl, H)
        dh = F.lmhead_backward(h, w[rank * Vl:(rank + 1) * Vl], labels, 1.0, lse, ent, g_lp, g_ent, dw, vocab_start=rank * Vl).float()
        dist.all_reduce(dh)
        dw_r = torch.zeros(V, H)
        dh_r = F.lmhead_backward(h, w, labels, 1.0, lse_r, ent_r, g_lp, g_ent, dw_r).float()
        ok_bwd = torch.allclose(dh, dh_r, atol=1e-5) and torch.allclose(dw, dw_r[rank * Vl:(rank + 1) * Vl], atol=1e-5)
        # distillation KL on slices vs full logits
        local = (h @ w[rank * Vl:(rank + 1) * Vl].t()).requires_grad_(True)
        loss, s_mass, _ = compute_forward_kl_topk_vocab_parallel(local, t_lp, t_ids, rank * Vl, dist.group.WORLD)
        loss.sum().backward()
        full = (h @ w.t()).requires_grad_(True)
        s = torch.log_softmax(full, -1).gather(-1, t_ids).clamp(min=-10)
        t = t_lp.clamp(min=-10)
        s_n, t_n = s - torch.logsumexp(s, -1, keepdim=True), t - torch.logsumexp(t, -1, keepdim=True)
        ref = (t_n.exp() * (t_n - s_n)).sum(-1)
        ref.sum().backward()
        ok_kl = torch.allclose(loss, ref, atol=1e-5) and torch.allclose(local.grad, full.grad[:, rank * Vl:(rank + 1) * Vl], atol=1e-5)
        q.put((rank, {"head": ok_head, "bwd": ok_bwd, "kl": ok_kl}))
        dist.destroy_process_group()
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_vocab_parallel_head_and_distillation_kl_on_gloo():
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_vp_proc, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    for r in range(2):
        assert "error" not in res[r], res[r]["error"]
        assert res[r] == {"head": True, "bwd": True, "kl": True}, res[r]


def test_separation_tables():
    from verl_b200.experimental.separation.utils import create_resource_pool_manager, create_role_worker_mapping
    from verl_b200.trainer.ppo.utils import Role

    cfg = {"trainer": {"nnodes": 1, "n_gpus_per_node": 4}, "rollout": {"nnodes": 1, "n_gpus_per_node": 2},
           "algorithm": {"adv_estimator": "grpo", "use_kl_in_reward": False},
           "actor_rollout_ref": {"actor": {"use_kl_loss": True}}, "critic": {"enable": None}}
    rpm = create_resource_pool_manager(cfg, [Role.Actor, Role.Rollout, Role.RefPolicy])
    assert rpm.resource_pool_spec == {"trainer_pool": [4], "rollout_pool": [2]} and rpm.get_n_gpus() == 6
    assert rpm.mapping[Role.Rollout] == "rollout_pool" and rpm.mapping[Role.RefPolicy] == "trainer_pool"


def test_linear_cross_entropy_autograd_matches_plain_torch():
    from verl_b200.utils.experimental.torch_functional import FusedLinearForPPO
    from verl_b200.utils.kernel import linear_cross_entropy

    g = torch.Generator().manual_seed(0)
    h = torch.randn(2, 5, 16, generator=g, requires_grad=True)
    w = (torch.randn(40, 16, generator=g) * 0.3).requires_grad_(True)
    y = torch.randint(0, 40, (2, 5), generator=g)
    lp, ent = linear_cross_entropy(h, w, y, temperature=0.7)
    (lp.sum() * 1.3 + ent.sum() * 0.4).backward()
    h2, w2 = h.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    logits = (h2 @ w2.t()) / 0.7
    ls = torch.log_softmax(logits, -1)
    lp_r = ls.gather(-1, y.unsqueeze(-1)).squeeze(-1)
    ent_r = -(ls.exp() * ls).sum(-1)
    (lp_r.sum() * 1.3 + ent_r.sum() * 0.4).backward()
    assert torch.allclose(lp, lp_r, atol=1e-5) and torch.allclose(ent, ent_r, atol=1e-5)
    assert torch.allclose(h.grad, h2.grad, atol=1e-5) and torch.allclose(w.grad, w2.grad, atol=1e-5)
    m_lp, _ = linear_cross_entropy(h.detach(), w.detach(), y, 0.7, "mean")
    assert torch.allclose(m_lp, lp_r.mean(), atol=1e-5)
    lp2, ent2 = FusedLinearForPPO()(h.detach(), w.detach(), y, 0.7)
    assert torch.allclose(lp2, lp_r, atol=1e-5) and lp2.shape == (2, 5)


def test_reward_config_dataclasses_check_the_manager_name():
    import pytest

    from verl_b200.workers.config.reward import RewardConfig, RewardManagerConfig, SandboxFusionConfig

    c = RewardConfig()
    assert c.reward_manager.name == "naive" and c.sandbox_fusion.max_concurrent == 64 and not c.reward_model.enable
    assert RewardManagerConfig(name="dapo").name == "dapo" and RewardManagerConfig(name="rate_limited").source == "register"
    with pytest.raises(ValueError, match="not registered"):
        RewardManagerConfig(name="no_such_manager")
    with pytest.raises(ValueError, match="module.path"):
        RewardManagerConfig(source="importlib", name="Mine")
    assert RewardManagerConfig(source="importlib", name="Mine", module={"path": "/x/y.py"}).module["path"] == "/x/y.py"
    with pytest.raises(ValueError, match="unknown reward manager source"):
        RewardManagerConfig(source="http")
    assert SandboxFusionConfig(url="http://s").url == "http://s"
