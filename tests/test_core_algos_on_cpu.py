"""Advantage estimators, losses and KL penalties against closed-form expectations."""
import numpy as np
import pytest
import torch

from verl_b200.trainer.ppo import core_algos as ca
from verl_b200.utils import torch_functional as VF


def test_registries():
    assert ca.get_adv_estimator_fn("grpo") is ca.compute_grpo_outcome_advantage
    assert ca.get_adv_estimator_fn(ca.AdvantageEstimator.GAE) is ca.compute_gae_advantage_return
    assert len(ca.ADV_ESTIMATOR_REGISTRY) == 14
    for n in ["vanilla", "dppo_tv", "dppo_kl", "gspo", "sapo", "gpg", "clip_cov", "kl_cov", "geo_mean", "dro", "cispo", "bypass_mode"]:
        assert callable(ca.get_policy_loss_fn(n))
    with pytest.raises(ValueError):
        ca.get_policy_loss_fn("nope")


def test_grpo_matches_manual_and_vectorized():
    torch.manual_seed(0)
    r = torch.zeros(6, 4)
    r[:, -1] = torch.tensor([1.0, 0.0, 0.5, 2.0, 2.0, 7.0])
    m = torch.ones(6, 4)
    m[1, 2:] = 0
    idx = np.array(["a", "a", "a", "b", "b", "c"], dtype=object)
    adv, ret = ca.compute_grpo_outcome_advantage(r, m, idx)
    a = torch.tensor([1.0, 0.0, 0.5])
    exp_a = (a - a.mean()) / (a.std() + 1e-6)
    assert torch.allclose(adv[:3, 0], exp_a, atol=1e-6)
    assert torch.allclose(adv[3:5, 0], torch.zeros(2))  # equal scores -> 0
    assert adv[5, 0].item() == pytest.approx(7.0, rel=1e-5)  # singleton: mean 0, std 1
    assert adv[1, 3].item() == 0.0 and torch.equal(adv, ret)
    adv2, _ = ca.compute_grpo_vectorized_outcome_advantage(r, m, idx)
    assert torch.allclose(adv, adv2, atol=1e-6)
    adv3, _ = ca.compute_grpo_outcome_advantage(r, m, idx, norm_adv_by_std_in_grpo=False)
    assert torch.allclose(adv3[:3, 0], a - a.mean(), atol=1e-6)


def test_rloo_and_variants():
    r = torch.zeros(4, 2)
    r[:, -1] = torch.tensor([1.0, 3.0, 5.0, 10.0])
    m = torch.ones(4, 2)
    idx = np.array([0, 0, 0, 1])
    adv, _ = ca.compute_rloo_outcome_advantage(r, m, idx)
    assert torch.allclose(adv[:3, 0], torch.tensor([1 - 4.0, 3 - 3.0, 5 - 2.0]))
    assert adv[3, 0].item() == 10.0
    adv2, _ = ca.compute_rloo_vectorized_outcome_advantage(r, m, idx)
    assert torch.allclose(adv, adv2)


def test_gae_reference_loop():
    torch.manual_seed(1)
    B, L = 3, 7
    r, v = torch.randn(B, L), torch.randn(B, L)
    m = torch.ones(B, L)
    m[0, 5:] = 0
    m[2, 2] = 0  # an observation token inside the sequence
    g, lam = 0.99, 0.95
    adv, ret = ca.compute_gae_advantage_return(r, v, m, g, lam)
    nv = torch.zeros(B)
    last = torch.zeros(B)
    raw = torch.zeros(B, L)
    for t in reversed(range(L)):
        delta = r[:, t] + g * nv - v[:, t]
        cand = delta + g * lam * last
        nv = v[:, t] * m[:, t] + (1 - m[:, t]) * nv
        last = cand * m[:, t] + (1 - m[:, t]) * last
        raw[:, t] = last
    assert torch.allclose(ret, raw + v, atol=1e-6)
    assert torch.allclose(adv, VF.masked_whiten(raw, m), atol=1e-5)


def test_reinforce_pp_remax_opo_gpg_passk():
    r = torch.zeros(4, 3)
    r[:, -1] = torch.tensor([1.0, 0.0, 1.0, 0.0])
    m = torch.ones(4, 3)
    idx = np.array([0, 0, 1, 1])
    a, ret = ca.compute_reinforce_plus_plus_outcome_advantage(r, m, gamma=0.5)
    assert torch.allclose(ret[0], torch.tensor([0.25, 0.5, 1.0]))
    a, ret = ca.compute_remax_outcome_advantage(r, torch.tensor([0.5, 0.5, 0.0, 0.0]), m)
    assert torch.allclose(ret[0], torch.ones(3)) and torch.allclose(a[0], torch.full((3,), 0.5))
    a, _ = ca.compute_opo_outcome_advantage(r, m, idx)
    assert torch.allclose(a[:, 0], torch.tensor([0.5, -0.5, 0.5, -0.5]))
    a, _ = ca.compute_gpg_outcome_advantage(r, m, idx)
    assert torch.allclose(a[:, 0], torch.tensor([1.0, -1.0, 1.0, -1.0]))  # alpha = 4/2
    a, _ = ca.compute_grpo_passk_outcome_advantage(r, m, idx, norm_adv_by_std_in_grpo=False)
    assert a[:, 0].tolist() == [1.0, 0.0, 1.0, 0.0]
    a, _ = ca.compute_reinforce_plus_plus_baseline_outcome_advantage(r, m, idx)
    assert a.shape == (4, 3) and abs(a.mean().item()) < 1e-6


def _otb_oracle(r, m, idx, olp, s2, isw=None, tail=True, eps=1e-8, compact=False):
    """Loop form of the optimal-token-baseline estimators, one group and one time step at a time."""
    bs, L = r.shape
    ret = torch.zeros(bs, L)
    W = torch.zeros(bs, L)
    for i in range(bs):
        acc = 0.0
        for t in reversed(range(L)):
            acc += float(r[i, t] * m[i, t])
            ret[i, t] = acc
        acc = 0.0
        for t in range(L):
            w = 1 - 2 * float(olp[i, t].exp()) + float(s2[i, t])
            if isw is not None:
                w *= float(isw[i, t]) ** 2
            acc += w * float(m[i, t])
            W[i, t] = acc
    pos = [[t for t in range(L) if m[i, t] > 0] for i in range(bs)]
    # frame: position t itself, or the t-th generated token when compacting
    frame = [pos[i] if compact else [t if m[i, t] > 0 else None for t in range(L)] for i in range(bs)]
    adv = torch.zeros(bs, L)
    groups = {}
    for i in range(bs):
        if compact and not pos[i]:
            continue
        groups.setdefault(idx[i], []).append(i)
    for members in groups.values():
        lens = sorted(len(pos[i]) for i in members)
        for i in members:
            for k, t in enumerate(frame[i]):
                if t is None:
                    continue
                base = 0.0
                if len(members) > 1:
                    num = den = 0.0
                    for j in members:
                        if k < len(frame[j]) and frame[j][k] is not None:
                            tj = frame[j][k]
                            num += float(ret[j, tj] * W[j, tj])
                            den += float(W[j, tj])
                    base = num / (den + eps)
                    if tail and len(pos[i]) == lens[-1] and lens[-1] > lens[-2] and k >= lens[-2]:
                        base = 0.0
                adv[i, t] = ret[i, t] - base
    return adv, ret


def _otb_case(seed, masks, idx):
    torch.manual_seed(seed)
    m = torch.tensor(masks, dtype=torch.float32)
    bs, L = m.shape
    r = torch.rand(bs, L) * m
    olp = -torch.rand(bs, L)
    s2 = torch.rand(bs, L) * 0.2
    isw = 0.5 + torch.rand(bs, L)
    return r, m, np.array(idx, dtype=object), olp, s2, isw


@pytest.mark.parametrize("tail", [True, False])
def test_optimal_token_baseline_matches_loop_form(tail):
    # ragged right-padded responses: a unique longest sample, a tie for longest, a singleton group
    masks = [[1, 1, 1, 1, 1, 1], [1, 1, 1, 0, 0, 0], [1, 1, 0, 0, 0, 0],
             [1, 1, 1, 1, 0, 0], [1, 1, 1, 1, 0, 0], [1, 0, 0, 0, 0, 0],
             [1, 1, 1, 1, 1, 0]]
    r, m, idx, olp, s2, isw = _otb_case(0, masks, ["a", "a", "a", "b", "b", "b", "solo"])
    for w in (None, isw):
        a, ret = ca.compute_optimal_token_baseline_advantage(r, m, idx, olp, s2, rollout_is_weights=w, handle_zero_tail=tail)
        a0, ret0 = _otb_oracle(r, m, list(idx), olp, s2, w, tail)
        assert torch.allclose(ret, ret0, atol=1e-5) and torch.allclose(a, a0, atol=1e-5)
    # singleton group: the advantage is the reward-to-go itself
    assert torch.allclose(a[6], ret[6] * m[6])
    # the unique longest sample of group "a" has baseline zero beyond the second-longest length
    if tail:
        assert torch.allclose(a[0, 3:], ret[0, 3:])


@pytest.mark.parametrize("tail", [True, False])
def test_multi_turn_optimal_token_baseline_matches_loop_form(tail):
    # tool / observation tokens (0) inside the trajectory, one sample with no generated token, one singleton group
    masks = [[1, 1, 0, 0, 1, 1, 1, 0], [1, 0, 0, 1, 1, 0, 0, 0], [1, 1, 1, 0, 0, 0, 1, 1],
             [0, 0, 0, 0, 0, 0, 0, 0], [1, 1, 0, 1, 0, 1, 0, 1], [1, 0, 1, 0, 0, 0, 0, 0]]
    r, m, idx, olp, s2, isw = _otb_case(1, masks, [0, 0, 0, 1, 1, 2])
    for w in (None, isw):
        a, ret = ca.compute_multi_turn_optimal_token_baseline_advantage(r, m, idx, olp, s2, rollout_is_weights=w,
                                                                        handle_zero_tail=tail)
        a0, ret0 = _otb_oracle(r, m, list(idx), olp, s2, w, tail, compact=True)
        assert torch.allclose(ret, ret0, atol=1e-5) and torch.allclose(a, a0, atol=1e-5)
    assert (a[3] == 0).all() and torch.allclose(a[4], ret[4] * m[4])  # group 1 has one sample with tokens
    assert (a * (1 - m) == 0).all()


def test_gdpo_whitens_over_tokens():
    torch.manual_seed(2)
    m = torch.tensor([[1, 1, 1, 1], [1, 0, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0]], dtype=torch.float32)
    r = torch.zeros(4, 4)
    r[torch.arange(4), (m.sum(-1) - 1).long()] = torch.tensor([1.0, 0.0, 0.5, 2.0])
    idx = np.array([0, 0, 1, 1])
    a, _ = ca.compute_gdpo_outcome_advantage(r, m, idx)
    g, _ = ca.compute_grpo_outcome_advantage(r, m, idx)
    want = VF.masked_whiten(g, m) * m
    assert torch.allclose(a, want, atol=1e-6)
    # two weighted components from the non-tensor batch
    nt = {"fmt": np.array([1.0, 0.0, 1.0, 0.0], dtype=np.float32), "acc": np.array([0.0, 1.0, 1.0, 3.0], dtype=np.float32)}
    a2, _ = ca.compute_gdpo_outcome_advantage(r, m, idx, config={"gdpo_reward_keys": ["fmt", "acc"], "gdpo_reward_weights": [0.5, 2.0]},
                                              non_tensor_batch=nt, batch={})
    comb = torch.zeros(4, 4)
    for w, k in ((0.5, "fmt"), (2.0, "acc")):
        rk = torch.zeros(4, 4)
        rk[:, 0] = torch.from_numpy(nt[k])
        comb = comb + w * ca.compute_grpo_outcome_advantage(rk, m, idx)[0]
    assert torch.allclose(a2, VF.masked_whiten(comb, m) * m, atol=1e-6)


@pytest.mark.parametrize("mode", ["token-mean", "token-sum", "seq-mean-token-sum", "seq-mean-token-mean", "seq-mean-token-sum-norm"])
def test_agg_loss_dp_invariance(mode):
    """Mean over DP ranks of the per-rank loss equals the single-process loss on the full batch."""
    torch.manual_seed(0)
    loss = torch.randn(8, 6)
    mask = (torch.rand(8, 6) > 0.3).float()
    mask[3] = 0
    full = ca.agg_loss(loss, mask, mode)
    info = dict(dp_size=2, batch_num_tokens=mask.sum(), global_batch_size=(mask.sum(-1) > 0).float().sum())
    parts = [ca.agg_loss(loss[i * 4:(i + 1) * 4], mask[i * 4:(i + 1) * 4], mode, **info) for i in range(2)]
    assert torch.allclose(sum(parts) / 2, full, atol=1e-6)
    with pytest.raises(ValueError):
        ca.agg_loss(loss, mask, "bogus")


def test_vanilla_policy_loss_clip_and_dual_clip():
    old = torch.zeros(1, 4)
    lp = torch.log(torch.tensor([[1.5, 0.5, 5.0, 1.0]]))
    adv = torch.tensor([[1.0, 1.0, -1.0, -1.0]])
    m = torch.ones(1, 4)
    loss, met = ca.compute_policy_loss_vanilla(old, lp, adv, m, "token-mean", dict(clip_ratio=0.2, clip_ratio_c=3.0))
    # token0: clipped at 1.2 -> -1.2 ; token1: -0.5 ; token2: A<0 ratio 5 -> max(5, 1.2)=5 then min(3, 5)=3 ; token3: 1
    assert loss.item() == pytest.approx((-1.2 - 0.5 + 3.0 + 1.0) / 4, rel=1e-5)
    assert met["actor/pg_clipfrac"] == pytest.approx(0.25) and met["actor/pg_clipfrac_lower"] == pytest.approx(0.25)
    l2, c, k, cl = ca.compute_policy_loss(old, lp, adv, m, cliprange=0.2)
    assert l2.item() == pytest.approx(loss.item())


def test_policy_losses_backward_and_is_weights():
    torch.manual_seed(0)
    old = -torch.rand(4, 5)
    adv = torch.randn(4, 5)
    m = (torch.rand(4, 5) > 0.2).float()
    cfg = dict(clip_ratio=0.2, policy_loss=dict(dro_beta=0.1))
    for name in ["vanilla", "dppo_tv", "dppo_kl", "gspo", "sapo", "gpg", "clip_cov", "kl_cov", "geo_mean", "dro", "cispo"]:
        lp = (old + 0.1 * torch.randn(4, 5)).requires_grad_(True)
        loss, met = ca.get_policy_loss_fn(name)(old, lp, adv, m, "token-mean", cfg, rollout_is_weights=torch.ones(4, 5))
        loss.backward()
        assert torch.isfinite(loss) and lp.grad is not None and torch.isfinite(lp.grad).all(), name
        assert (lp.grad * (1 - m)).abs().sum() == 0 or name in ("gspo", "geo_mean"), name


def test_kl_penalty_estimators():
    lp, ref = torch.tensor([0.0, -1.0]), torch.tensor([-0.5, -0.2])
    assert torch.allclose(ca.kl_penalty(lp, ref, "kl"), lp - ref)
    assert torch.allclose(ca.kl_penalty(lp, ref, "abs"), (lp - ref).abs())
    assert torch.allclose(ca.kl_penalty(lp, ref, "mse"), 0.5 * (lp - ref) ** 2)
    k = ref - lp
    assert torch.allclose(ca.kl_penalty(lp, ref, "low_var_kl"), torch.exp(k) - k - 1)
    x = lp.clone().requires_grad_(True)
    ca.kl_penalty(x, ref, "k3+").sum().backward()
    assert torch.allclose(x.grad, lp - ref)  # straight-through: k2 gradient
    with pytest.raises(NotImplementedError):
        ca.kl_penalty(lp, ref, "full")


def test_value_loss_and_kl_controllers():
    v, ret, old = torch.tensor([[1.0, 3.0]]), torch.tensor([[0.0, 0.0]]), torch.tensor([[0.0, 0.0]])
    loss, frac = ca.compute_value_loss(v, ret, old, torch.ones(1, 2), cliprange_value=0.5)
    assert loss.item() == pytest.approx(0.5 * (1.0 + 9.0) / 2) and frac.item() == 0.0
    c = ca.get_kl_controller(dict(type="adaptive", kl_coef=0.1, target_kl=0.1, horizon=100))
    c.update(0.2, 10)
    assert c.value == pytest.approx(0.1 * (1 + 0.2 * 10 / 100))
    f = ca.get_kl_controller(dict(type="fixed", kl_coef=0.3))
    f.update(9, 9)
    assert f.value == 0.3


def test_masked_ops():
    x = torch.tensor([[1.0, float("nan")], [3.0, 5.0]])
    m = torch.tensor([[1.0, 0.0], [1.0, 1.0]])
    assert VF.masked_mean(x, m).item() == pytest.approx(3.0)
    assert VF.masked_var(torch.tensor([1.0, 3.0, 100.0]), torch.tensor([1.0, 1.0, 0.0])).item() == pytest.approx(2.0)
    with pytest.raises(ValueError):
        VF.masked_var(torch.ones(2), torch.tensor([1.0, 0.0]))
    rm = VF.get_response_mask(torch.tensor([[5, 2, 7, 2], [1, 1, 1, 1]]), eos_token=2)
    assert rm.tolist() == [[1, 1, 0, 0], [1, 1, 1, 1]]
