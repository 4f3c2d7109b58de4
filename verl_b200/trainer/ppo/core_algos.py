"""Advantage estimators, policy losses, KL penalties and loss aggregation for PPO-family algorithms.

Pure tensor math (runs on CPU or GPU tensors alike); the device kernels in ``verl_b200.ops`` implement
the two hot estimators (GRPO, GAE) natively and are checked against the functions in this file.

API parity target: ``verl/trainer/ppo/core_algos.py`` — registries (:53-150), KL controllers (:153-213),
the 14 advantage estimators (:216-1120), ``agg_loss`` (:1140), the policy-loss family (:1285-2548),
``compute_value_loss`` (:2124), ``kl_penalty`` (:2187), ``compute_pf_ppo_reweight_data`` (:2253).
"""

from __future__ import annotations

from collections import defaultdict
from enum import Enum
from typing import Any, Callable, Optional

import numpy as np
import torch

from ...utils import torch_functional as VF

__all__ = [
    "register_policy_loss", "get_policy_loss_fn", "AdvantageEstimator", "register_adv_est", "get_adv_estimator_fn",
    "AdaptiveKLController", "FixedKLController", "get_kl_controller", "compute_gae_advantage_return",
    "compute_grpo_outcome_advantage", "compute_grpo_vectorized_outcome_advantage", "compute_gdpo_outcome_advantage",
    "compute_grpo_passk_outcome_advantage", "compute_reinforce_plus_plus_baseline_outcome_advantage",
    "compute_rloo_outcome_advantage", "compute_opo_outcome_advantage", "compute_reinforce_plus_plus_outcome_advantage",
    "compute_remax_outcome_advantage", "compute_gpg_outcome_advantage", "compute_rloo_vectorized_outcome_advantage",
    "compute_optimal_token_baseline_advantage", "compute_multi_turn_optimal_token_baseline_advantage",
    "compute_rewards", "agg_loss", "compute_policy_loss", "compute_policy_loss_vanilla", "compute_entropy_loss",
    "compute_value_loss", "kl_penalty", "kl_penalty_forward", "compute_pf_ppo_reweight_data",
]

PolicyLossFn = Callable[..., tuple[torch.Tensor, dict[str, Any]]]

# ----------------------------------------------------------------------------------------------- registries
POLICY_LOSS_REGISTRY: dict[str, PolicyLossFn] = {}
ADV_ESTIMATOR_REGISTRY: dict[str, Callable] = {}


def register_policy_loss(name: str):
    def deco(fn: PolicyLossFn) -> PolicyLossFn:
        POLICY_LOSS_REGISTRY[name] = fn
        return fn

    return deco


def get_policy_loss_fn(name: str) -> PolicyLossFn:
    if name not in POLICY_LOSS_REGISTRY:
        raise ValueError(f"Unsupported loss mode: {name}. Supported modes are: {sorted(POLICY_LOSS_REGISTRY)}")
    return POLICY_LOSS_REGISTRY[name]


class AdvantageEstimator(str, Enum):
    GAE = "gae"
    GRPO = "grpo"
    REINFORCE_PLUS_PLUS = "reinforce_plus_plus"
    REINFORCE_PLUS_PLUS_BASELINE = "reinforce_plus_plus_baseline"
    REMAX = "remax"
    RLOO = "rloo"
    OPO = "opo"
    GRPO_PASSK = "grpo_passk"
    GPG = "gpg"
    RLOO_VECTORIZED = "rloo_vectorized"
    GRPO_VECTORIZED = "grpo_vectorized"
    OPTIMAL_TOKEN_BASELINE = "optimal_token_baseline"
    TIR_OPTIMAL_TOKEN_BASELINE = "tir_optimal_token_baseline"
    GDPO = "gdpo"


def _est_name(x) -> str:
    return x.value if isinstance(x, Enum) else str(x)


def register_adv_est(name_or_enum):
    def deco(fn):
        key = _est_name(name_or_enum)
        if key in ADV_ESTIMATOR_REGISTRY and ADV_ESTIMATOR_REGISTRY[key] is not fn:
            raise ValueError(f"Adv estimator {key} has already been registered")
        ADV_ESTIMATOR_REGISTRY[key] = fn
        return fn

    return deco


def get_adv_estimator_fn(name_or_enum):
    key = _est_name(name_or_enum)
    if key not in ADV_ESTIMATOR_REGISTRY:
        raise ValueError(f"Unknown advantage estimator simply: {key}")
    return ADV_ESTIMATOR_REGISTRY[key]


# ----------------------------------------------------------------------------------------------- KL control
class AdaptiveKLController:
    """Proportional controller on the KL coefficient (Ziegler et al., 2019)."""

    def __init__(self, init_kl_coef: float, target_kl: float, horizon: int):
        self.value = init_kl_coef
        self.target = target_kl
        self.horizon = horizon

    def update(self, current_kl: float, n_steps: int) -> None:
        err = float(np.clip(current_kl / self.target - 1.0, -0.2, 0.2))
        self.value *= 1.0 + err * n_steps / self.horizon


class FixedKLController:
    def __init__(self, kl_coef: float):
        self.value = kl_coef

    def update(self, current_kl: float, n_steps: int) -> None:
        return None


def get_kl_controller(kl_ctrl):
    kind = kl_ctrl.type if hasattr(kl_ctrl, "type") else kl_ctrl["type"]
    get = (lambda k: getattr(kl_ctrl, k)) if hasattr(kl_ctrl, "type") else (lambda k: kl_ctrl[k])
    if kind == "fixed":
        return FixedKLController(kl_coef=get("kl_coef"))
    if kind == "adaptive":
        assert get("horizon") > 0, f"horizon must be larger than 0. Got {get('horizon')}"
        return AdaptiveKLController(init_kl_coef=get("kl_coef"), target_kl=get("target_kl"), horizon=get("horizon"))
    raise NotImplementedError(kind)


# ----------------------------------------------------------------------------------------------- group helpers
def _group_ids(index) -> tuple[torch.Tensor, int]:
    """Map arbitrary hashable per-sample ids to dense int64 group ids."""
    table: dict[Any, int] = {}
    out = []
    for v in (index.tolist() if isinstance(index, (np.ndarray, torch.Tensor)) else list(index)):
        out.append(table.setdefault(v, len(table)))
    return torch.tensor(out, dtype=torch.int64), len(table)


def _group_mean_std(scores: torch.Tensor, gid: torch.Tensor, ng: int, unbiased: bool = True):
    """Per-sample (mean, std, count) of its group; singleton groups get mean 0 / std 1."""
    gid = gid.to(scores.device)
    ones = torch.ones_like(scores)
    cnt = torch.zeros(ng, dtype=scores.dtype, device=scores.device).index_add_(0, gid, ones)
    s1 = torch.zeros(ng, dtype=scores.dtype, device=scores.device).index_add_(0, gid, scores)
    mean = s1 / cnt.clamp(min=1)
    dev2 = torch.zeros(ng, dtype=scores.dtype, device=scores.device).index_add_(0, gid, (scores - mean[gid]) ** 2)
    denom = (cnt - 1).clamp(min=1) if unbiased else cnt.clamp(min=1)
    std = torch.sqrt(dev2 / denom)
    single = cnt <= 1
    mean = torch.where(single, torch.zeros_like(mean), mean)
    std = torch.where(single, torch.ones_like(std), std)
    return mean[gid], std[gid], cnt[gid]


# ----------------------------------------------------------------------------------------------- estimators
@register_adv_est(AdvantageEstimator.GAE)
def compute_gae_advantage_return(token_level_rewards, values, response_mask, gamma, lam):
    """Generalised advantage estimation with mask carry-through, then batch whitening of the advantages."""
    with torch.no_grad():
        L = token_level_rewards.shape[-1]
        next_v = torch.zeros_like(values[:, 0])
        run = torch.zeros_like(values[:, 0])
        adv = torch.zeros_like(values)
        for t in range(L - 1, -1, -1):
            m = response_mask[:, t]
            delta = token_level_rewards[:, t] + gamma * next_v - values[:, t]
            cand = delta + gamma * lam * run
            next_v = values[:, t] * m + (1 - m) * next_v
            run = cand * m + (1 - m) * run
            adv[:, t] = run
        returns = adv + values
        adv = VF.masked_whiten(adv, response_mask)
    return adv, returns


@register_adv_est(AdvantageEstimator.GRPO)
def compute_grpo_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                   norm_adv_by_std_in_grpo: bool = True, config=None):
    """Outcome advantage normalised inside each prompt group (``index`` holds the group id per sample)."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        gid, ng = _group_ids(index)
        mean, std, _ = _group_mean_std(scores, gid, ng)
        a = (scores - mean) / (std + epsilon) if norm_adv_by_std_in_grpo else scores - mean
        a = a.unsqueeze(-1) * response_mask
    return a, a


@register_adv_est(AdvantageEstimator.GRPO_VECTORIZED)
def compute_grpo_vectorized_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                              norm_adv_by_std_in_grpo: bool = True, config=None):
    """Same estimator as GRPO, computed with segment reductions on the tensor's own device."""
    from ...utils.groupwise import as_torch_index, group_mean_std

    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        g = as_torch_index(index, device=scores.device)
        mean_g, std_g, _ = group_mean_std(scores, g)
        a = (scores - mean_g[g]) / (std_g[g] + epsilon) if norm_adv_by_std_in_grpo else scores - mean_g[g]
        a = a.unsqueeze(-1) * response_mask
    return a, a


@register_adv_est(AdvantageEstimator.GDPO)
def compute_gdpo_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                   norm_adv_by_std_in_grpo: bool = True, config=None, non_tensor_batch=None,
                                   batch=None, **kwargs):
    """Group-decoupled normalisation: every reward component is group-normalised on its own, the
    normalised components are combined with their weights, and the sum is whitened over the batch."""
    with torch.no_grad():
        keys = list(getattr(config, "gdpo_reward_keys", None) or (config.get("gdpo_reward_keys") if isinstance(config, dict) else None) or [])
        weights = list(getattr(config, "gdpo_reward_weights", None) or (config.get("gdpo_reward_weights") if isinstance(config, dict) else None) or [])
        gid, ng = _group_ids(index)
        comps = []
        if keys and non_tensor_batch is not None and all(k in non_tensor_batch for k in keys):
            for k in keys:
                comps.append(torch.as_tensor(np.asarray(non_tensor_batch[k], dtype=np.float32), device=response_mask.device))
        else:
            comps.append(token_level_rewards.sum(-1))
        if not weights:
            weights = [1.0] * len(comps)
        total = torch.zeros_like(comps[0])
        for w, c in zip(weights, comps):
            mean, std, _ = _group_mean_std(c, gid, ng)
            total = total + w * ((c - mean) / (std + epsilon) if norm_adv_by_std_in_grpo else (c - mean))
        # whitened over tokens, so longer responses weigh more in the batch statistics (as the reference does)
        a = VF.masked_whiten(total.unsqueeze(-1) * response_mask, response_mask) * response_mask
    return a, a


@register_adv_est(AdvantageEstimator.GRPO_PASSK)
def compute_grpo_passk_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                         norm_adv_by_std_in_grpo: bool = True, config=None, **kwargs):
    """Pass@k GRPO: only the best sample of each group gets a non-zero advantage (best - second best)."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        adv = torch.zeros_like(scores)
        groups = defaultdict(list)
        for i, g in enumerate(index.tolist() if hasattr(index, "tolist") else index):
            groups[g].append(i)
        for g, ids in groups.items():
            if len(ids) < 2:
                raise ValueError(f"Pass@k requires at least 2 samples per group. Got {len(ids)} for group {g}.")
            r = scores[ids]
            top, pos = torch.topk(r, 2)
            a = top[0] - top[1]
            if norm_adv_by_std_in_grpo:
                a = a / (r.std() + epsilon)
            adv[ids[int(pos[0])]] = a
        adv = adv.unsqueeze(-1) * response_mask
    return adv, adv


@register_adv_est(AdvantageEstimator.REINFORCE_PLUS_PLUS_BASELINE)
def compute_reinforce_plus_plus_baseline_outcome_advantage(token_level_rewards, response_mask, index,
                                                           epsilon: float = 1e-6, config=None, **kwargs):
    """Group-mean baseline, then whitening of the token-level advantages over the batch."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        gid, ng = _group_ids(index)
        mean, _, _ = _group_mean_std(scores, gid, ng)
        a = (scores - mean).unsqueeze(-1) * response_mask
        a = VF.masked_whiten(a, response_mask) * response_mask
    return a, a


@register_adv_est(AdvantageEstimator.RLOO)
def compute_rloo_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6, config=None,
                                   **kwargs):
    """Leave-one-out baseline: A_i = n/(n-1) * (r_i - mean_group)."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        gid, ng = _group_ids(index)
        mean, _, cnt = _group_mean_std(scores, gid, ng)
        f = torch.where(cnt > 1, cnt / (cnt - 1).clamp(min=1), torch.ones_like(cnt))
        a = torch.where(cnt > 1, f * (scores - mean), scores)
        a = a.unsqueeze(-1) * response_mask
    return a, a


@register_adv_est(AdvantageEstimator.RLOO_VECTORIZED)
def compute_rloo_vectorized_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                              config=None, **kwargs):
    from ...utils.groupwise import as_torch_index

    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        g = as_torch_index(index, device=scores.device)
        ng = int(g.max().item()) + 1 if g.numel() else 0
        cnt = torch.bincount(g, minlength=ng).to(scores.dtype)
        tot = torch.zeros(ng, dtype=scores.dtype, device=scores.device).index_add_(0, g, scores)
        n = cnt[g]
        loo = (tot[g] - scores) / (n - 1).clamp(min=1)
        a = torch.where(n > 1, scores - loo, scores)
        a = a.unsqueeze(-1) * response_mask
    return a, a


@register_adv_est(AdvantageEstimator.OPO)
def compute_opo_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6, config=None,
                                  **kwargs):
    """Optimal (length-weighted) baseline per group: b = sum(len_i * r_i) / sum(len_i)."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        lens = response_mask.sum(dim=-1)
        gid, ng = _group_ids(index)
        gid = gid.to(scores.device)
        num = torch.zeros(ng, dtype=scores.dtype, device=scores.device).index_add_(0, gid, lens * scores)
        den = torch.zeros(ng, dtype=scores.dtype, device=scores.device).index_add_(0, gid, lens)
        cnt = torch.bincount(gid, minlength=ng)
        base = torch.where(cnt > 1, num / den.clamp(min=1e-8), torch.zeros_like(num))
        a = (scores - base[gid]).unsqueeze(-1) * response_mask
    return a, a


@register_adv_est(AdvantageEstimator.REINFORCE_PLUS_PLUS)
def compute_reinforce_plus_plus_outcome_advantage(token_level_rewards, response_mask, config=None, gamma=None,
                                                  **kwargs):
    """Discounted return-to-go (reset across masked tokens), whitened over the batch."""
    if gamma is None:
        gamma = config.gamma if hasattr(config, "gamma") else (config.get("gamma", 1.0) if config else 1.0)
    with torch.no_grad():
        returns = torch.zeros_like(token_level_rewards)
        run = torch.zeros_like(token_level_rewards[:, 0])
        for t in range(token_level_rewards.shape[1] - 1, -1, -1):
            run = token_level_rewards[:, t] + gamma * run
            returns[:, t] = run
            run = run * response_mask[:, t]
        a = VF.masked_whiten(returns, response_mask) * response_mask
    return a, returns


@register_adv_est(AdvantageEstimator.REMAX)
def compute_remax_outcome_advantage(token_level_rewards, reward_baselines, response_mask, config=None, **kwargs):
    """Return-to-go minus the reward of the greedy rollout of the same prompt."""
    with torch.no_grad():
        returns = (token_level_rewards * response_mask).flip(-1).cumsum(-1).flip(-1)
        a = returns - reward_baselines.unsqueeze(-1) * response_mask
    return a, returns


@register_adv_est(AdvantageEstimator.GPG)
def compute_gpg_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6, f_norm: float = 1.0,
                                  config=None, **kwargs):
    """Group policy gradient: group-mean baseline scaled by batch_size / #samples with non-zero reward."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        gid, ng = _group_ids(index)
        mean, _, _ = _group_mean_std(scores, gid, ng)
        m = torch.count_nonzero(scores)
        alpha = scores.shape[0] / m.clamp(min=1)
        a = alpha * (scores - mean) / f_norm
        a = a.unsqueeze(-1) * response_mask
    return a, a


def _otb_baselines(returns, W, valid, gid, ng, lengths, epsilon, handle_zero_tail):
    """Per-timestep baseline of every sample's group on an aligned [bs, L] frame.

    ``valid`` marks the positions that vote: B_g(t) = sum_{i in g} G_i(t) W_i(t) valid_i(t) / (sum W_i(t) valid_i(t) + eps).
    Groups of one sample get baseline zero (the advantage is the return). With ``handle_zero_tail`` the unique
    longest sample of a group gets baseline zero beyond the length of the second longest: only it votes there."""
    bs, L = returns.shape
    dev = returns.device
    gid = gid.to(dev)
    Wv = W * valid
    num = torch.zeros(ng, L, dtype=returns.dtype, device=dev).index_add_(0, gid, returns * Wv)
    den = torch.zeros(ng, L, dtype=returns.dtype, device=dev).index_add_(0, gid, Wv)
    base = (num / (den + epsilon))[gid]
    count = torch.zeros(ng, dtype=torch.long, device=dev).index_add_(0, gid, torch.ones(bs, dtype=torch.long, device=dev))
    base = base * (count[gid] > 1).unsqueeze(-1)
    if handle_zero_tail and bs > 0:
        lengths = lengths.to(dev).long()
        # longest and second-longest length per group (counting multiplicity), without a Python loop over groups
        top = torch.zeros(ng, dtype=torch.long, device=dev).scatter_reduce_(0, gid, lengths, reduce="amax", include_self=True)
        n_top = torch.zeros(ng, dtype=torch.long, device=dev).index_add_(0, gid, (lengths == top[gid]).long())
        rest = torch.where(lengths == top[gid], torch.zeros_like(lengths), lengths)
        second = torch.zeros(ng, dtype=torch.long, device=dev).scatter_reduce_(0, gid, rest, reduce="amax", include_self=True)
        lone = (lengths == top[gid]) & (n_top[gid] == 1) & (count[gid] > 1) & (top[gid] > second[gid])
        pos = torch.arange(L, device=dev).unsqueeze(0)
        base = torch.where(lone.unsqueeze(-1) & (pos >= second[gid].unsqueeze(-1)), torch.zeros_like(base), base)
    return base


def _otb_inputs(token_level_rewards, response_mask, old_log_probs, sum_pi_squared, rollout_is_weights):
    """Reward-to-go returns and the cumulative path-variance proxy W_t = sum_{s<=t} (1 - 2 pi_s + sum pi_s^2) over
    generated tokens (times the squared truncated importance weight when rollout correction is on)."""
    returns = (token_level_rewards * response_mask).flip(-1).cumsum(-1).flip(-1)
    w_step = 1.0 - 2.0 * torch.exp(old_log_probs) + sum_pi_squared
    if rollout_is_weights is not None:
        w_step = w_step * rollout_is_weights.pow(2)
    return returns, torch.cumsum(w_step * response_mask, dim=-1)


@register_adv_est(AdvantageEstimator.OPTIMAL_TOKEN_BASELINE)
def compute_optimal_token_baseline_advantage(token_level_rewards, response_mask, index, old_log_probs,
                                             sum_pi_squared, rollout_is_weights=None, handle_zero_tail: bool = True,
                                             epsilon: float = 1e-8, config=None, **kwargs):
    """Variance-optimal per-timestep baseline within each prompt group; returns (advantages, reward-to-go).

    Parity target: ``verl/trainer/ppo/core_algos.py:871-985``: finished samples leave both sums, a single-sample group
    keeps its return as the advantage, the tail rule uses the longest against the second-longest response."""
    with torch.no_grad():
        returns, W = _otb_inputs(token_level_rewards, response_mask, old_log_probs, sum_pi_squared, rollout_is_weights)
        gid, ng = _group_ids(index)
        base = _otb_baselines(returns, W, response_mask.to(returns.dtype), gid, ng, response_mask.sum(-1), epsilon,
                              handle_zero_tail)
        adv = (returns - base) * response_mask
    return adv, returns


@register_adv_est(AdvantageEstimator.TIR_OPTIMAL_TOKEN_BASELINE)
def compute_multi_turn_optimal_token_baseline_advantage(token_level_rewards, response_mask, index, old_log_probs,
                                                        sum_pi_squared, rollout_is_weights=None,
                                                        handle_zero_tail: bool = True, epsilon: float = 1e-8,
                                                        config=None, **kwargs):
    """Multi-turn variant: tool / observation tokens (mask 0 inside the trajectory) neither accumulate variance nor
    receive an advantage, and the baseline is indexed by the number of generated tokens so far: the generated tokens
    of every sample are compacted to the left before the group statistics and scattered back afterwards. Samples
    without a generated token belong to no group. Parity target: ``verl/trainer/ppo/core_algos.py:988-1121``."""
    with torch.no_grad():
        returns, W = _otb_inputs(token_level_rewards, response_mask, old_log_probs, sum_pi_squared, rollout_is_weights)
        bs, L = returns.shape
        m = response_mask > 0
        lengths = m.sum(-1)
        # stable left-compaction: generated tokens first, in order
        order = torch.argsort((~m).to(torch.int8), dim=-1, stable=True)
        filled = (torch.arange(L, device=returns.device).unsqueeze(0) < lengths.unsqueeze(-1)).to(returns.dtype)
        c_ret = torch.gather(returns, 1, order) * filled
        c_W = torch.gather(W, 1, order) * filled
        keep = lengths > 0
        adv_c = torch.zeros_like(c_ret)
        if bool(keep.any()):
            idx_np = np.asarray(index, dtype=object)[keep.cpu().numpy()]
            gid, ng = _group_ids(idx_np)
            # every compacted position below the length votes; the frame is zero beyond it, as in the reference
            ones = torch.ones_like(c_ret[keep])
            base = _otb_baselines(c_ret[keep], c_W[keep], ones, gid, ng, lengths[keep], epsilon, handle_zero_tail)
            adv_c[keep] = c_ret[keep] - base
        adv = torch.zeros_like(returns).scatter_(1, order, adv_c * filled) * response_mask
    return adv, returns


# ----------------------------------------------------------------------------------------------- rewards / agg
def compute_rewards(token_level_scores, old_log_prob, ref_log_prob, kl_ratio):
    return token_level_scores - (old_log_prob - ref_log_prob) * kl_ratio


def agg_loss(loss_mat: torch.Tensor, loss_mask: torch.Tensor, loss_agg_mode: str, dp_size: int = 1,
             batch_num_tokens: Optional[int] = None, global_batch_size: Optional[int] = None,
             loss_scale_factor: Optional[int] = None) -> torch.Tensor:
    """Reduce a [bs, len] loss matrix to a scalar such that the data-parallel gradient *average* equals the
    requested aggregate over the *global* batch (hence the ``* dp_size`` factors)."""
    if loss_agg_mode == "token-mean":
        if batch_num_tokens is None:
            if dp_size > 1:
                raise ValueError("(global) batch_num_tokens is required when dp_size > 1")
            batch_num_tokens = loss_mask.sum()
        return VF.masked_sum(loss_mat, loss_mask) / batch_num_tokens * dp_size
    if loss_agg_mode == "token-sum":
        return VF.masked_sum(loss_mat, loss_mask) * dp_size
    if loss_agg_mode in ("seq-mean-token-sum", "seq-mean-token-sum-norm", "seq-mean-token-mean"):
        tok = loss_mask.sum(dim=-1)
        seq = (loss_mat * loss_mask).sum(dim=-1)
        if loss_agg_mode == "seq-mean-token-mean":
            seq = seq / (tok + 1e-8)
        alive = (tok > 0).float()
        if global_batch_size is None:
            if dp_size > 1:
                raise ValueError("global_batch_size is required when dp_size > 1")
            global_batch_size = alive.sum()
        loss = VF.masked_sum(seq, alive) / global_batch_size * dp_size
        if loss_agg_mode == "seq-mean-token-sum-norm":
            loss = loss / (loss_scale_factor if loss_scale_factor is not None else loss_mask.shape[-1])
        return loss
    raise ValueError(f"Invalid loss_agg_mode: {loss_agg_mode}")


# ----------------------------------------------------------------------------------------------- policy losses
def _cfg_get(config, key, default=None):
    if config is None:
        return default
    if hasattr(config, "get"):
        try:
            v = config.get(key, default)
            return default if v is None else v
        except TypeError:
            pass
    v = getattr(config, key, default)
    return default if v is None else v


def _clip_bounds(config):
    eps = _cfg_get(config, "clip_ratio", 0.2)
    lo = _cfg_get(config, "clip_ratio_low", eps)
    hi = _cfg_get(config, "clip_ratio_high", eps)
    return lo, hi


def _global_info(config) -> dict:
    info = _cfg_get(config, "global_batch_info", None)
    return dict(info) if info else {}


def _finish(pg_losses, response_mask, loss_agg_mode, config, rollout_is_weights, metrics: dict):
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    loss = agg_loss(loss_mat=pg_losses, loss_mask=response_mask, loss_agg_mode=loss_agg_mode, **_global_info(config))
    return loss, {k: (v.detach().item() if torch.is_tensor(v) else float(v)) for k, v in metrics.items()}


def _ratio(old_log_prob, log_prob, clamp: bool = True):
    lr = log_prob - old_log_prob
    if clamp:
        lr = torch.clamp(lr, min=-20.0, max=20.0)
    return lr, torch.exp(lr)


def compute_policy_loss(old_log_prob, log_prob, advantages, response_mask, cliprange=None, cliprange_low=None,
                        cliprange_high=None, clip_ratio_c: float = 3.0, loss_agg_mode: str = "token-mean"):
    """Legacy entry point (tuple return) kept for API compatibility."""
    cfg = dict(clip_ratio=cliprange, clip_ratio_low=cliprange_low, clip_ratio_high=cliprange_high,
               clip_ratio_c=clip_ratio_c)
    loss, m = compute_policy_loss_vanilla(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode, cfg)
    t = lambda k: torch.tensor(m[k], device=loss.device)
    return loss, t("actor/pg_clipfrac"), t("actor/ppo_kl"), t("actor/pg_clipfrac_lower")


@register_policy_loss("vanilla")
def compute_policy_loss_vanilla(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode: str = "token-mean",
                                config=None, rollout_is_weights=None):
    """PPO clipped surrogate with dual-clip (arXiv:1707.06347, arXiv:1912.09729)."""
    assert config is not None
    lo, hi = _clip_bounds(config)
    c = _cfg_get(config, "clip_ratio_c", 3.0)
    assert c > 1.0, f"The lower bound of the clip_ratio_c for dual-clip PPO should be greater than 1.0, but get the value: {c}."
    lr, ratio = _ratio(old_log_prob, log_prob)
    unclipped = -advantages * ratio
    clipped = -advantages * torch.clamp(ratio, 1 - lo, 1 + hi)
    first = torch.maximum(unclipped, clipped)
    floor = -advantages * c
    second = torch.minimum(floor, first)
    neg = advantages < 0
    losses = torch.where(neg, second, first)
    metrics = {
        "actor/pg_clipfrac": VF.masked_mean((clipped > unclipped).float(), response_mask),
        "actor/ppo_kl": VF.masked_mean(-lr, response_mask),
        "actor/pg_clipfrac_lower": VF.masked_mean((first > floor).float() * neg.float(), response_mask),
    }
    return _finish(losses, response_mask, loss_agg_mode, config, rollout_is_weights, metrics)


def _dppo(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode, config, rollout_is_weights, divergence):
    lo, hi = _clip_bounds(config)
    lr, ratio = _ratio(old_log_prob, log_prob)
    cap = _cfg_get(config, "clip_ratio_c", 20.0)
    w = torch.clamp(ratio, max=cap).detach()
    p, p_old = torch.exp(log_prob), torch.exp(old_log_prob)
    if divergence == "tv":
        ok_pos, ok_neg = (p - p_old) <= hi, (p - p_old) >= -lo
    else:
        bkl = p_old * (old_log_prob - log_prob) + (1 - p_old) * torch.log((1.0 - p_old + 1e-8) / (1.0 - p + 1e-8))
        ok_pos, ok_neg = (bkl <= hi) | (p <= p_old), (bkl <= lo) | (p >= p_old)
    keep = torch.where(advantages > 0, ok_pos, ok_neg).detach().float()
    losses = -advantages * w * log_prob * keep
    metrics = {
        "actor/pg_clipfrac": VF.masked_mean(1.0 - keep, response_mask),
        "actor/ppo_kl": VF.masked_mean(-lr, response_mask),
        "actor/pg_clipfrac_lower": VF.masked_mean((ratio > cap).float() * keep, response_mask),
    }
    return _finish(losses, response_mask, loss_agg_mode, config, rollout_is_weights, metrics)


@register_policy_loss("dppo_tv")
def compute_policy_loss_dppo_tv(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                                config=None, rollout_is_weights=None):
    """Divergence-PPO with a total-variation trust region on the token probability."""
    assert config is not None
    return _dppo(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode, config, rollout_is_weights, "tv")


@register_policy_loss("dppo_kl")
def compute_policy_loss_dppo_kl(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                                config=None, rollout_is_weights=None):
    """Divergence-PPO with a binary-KL trust region on the token probability."""
    assert config is not None
    return _dppo(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode, config, rollout_is_weights, "kl")


@register_policy_loss("gspo")
def compute_policy_loss_gspo(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="seq-mean-token-mean",
                             config=None, rollout_is_weights=None):
    """Group sequence policy optimisation: sequence-level (length-normalised) importance ratio with the
    token's own gradient re-attached."""
    assert config is not None
    lo, hi = _clip_bounds(config)
    lr = log_prob - old_log_prob
    n = response_mask.sum(-1).clamp(min=1)
    seq_lr = (lr * response_mask).sum(-1) / n
    log_s = torch.clamp(log_prob - log_prob.detach() + seq_lr.detach().unsqueeze(-1), max=10.0)
    s = torch.exp(log_s)
    a, b = -advantages * s, -advantages * torch.clamp(s, 1 - lo, 1 + hi)
    metrics = {
        "actor/pg_clipfrac": VF.masked_mean((b > a).float(), response_mask),
        "actor/ppo_kl": VF.masked_mean(-lr, response_mask),
        "actor/pg_clipfrac_lower": 0.0,
    }
    return _finish(torch.maximum(a, b), response_mask, "seq-mean-token-mean", config, rollout_is_weights, metrics)


@register_policy_loss("sapo")
def compute_policy_loss_sapo(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="seq-mean-token-mean",
                             config=None, rollout_is_weights=None):
    """Soft adaptive policy optimisation: sigmoid gate on the ratio instead of a hard clip."""
    assert config is not None
    tp = torch.as_tensor(_cfg_get(config, "tau_pos", 1.0), dtype=advantages.dtype, device=advantages.device)
    tn = torch.as_tensor(_cfg_get(config, "tau_neg", 1.05), dtype=advantages.dtype, device=advantages.device)
    lr, ratio = _ratio(old_log_prob, log_prob)
    tau = torch.where(advantages > 0, tp, tn)
    gate = torch.sigmoid(tau * (ratio - 1.0)) * (4.0 / tau)
    metrics = {"actor/pg_clipfrac": 0.0, "actor/ppo_kl": VF.masked_mean(-lr, response_mask),
               "actor/pg_clipfrac_lower": 0.0}
    return _finish(-gate * advantages, response_mask, "seq-mean-token-mean", config, rollout_is_weights, metrics)


@register_policy_loss("gpg")
def compute_policy_loss_gpg(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                            config=None, rollout_is_weights=None):
    assert config is not None
    return _finish(-log_prob * advantages, response_mask, loss_agg_mode, config, rollout_is_weights, {})


@register_policy_loss("clip_cov")
def compute_policy_loss_clip_cov(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                                 config=None, rollout_is_weights=None):
    """Clip-Cov (arXiv:2505.22617): drop the gradient of a random subset of high-covariance tokens."""
    assert config is not None
    pl = _cfg_get(config, "policy_loss", None)
    frac = _cfg_get(pl, "clip_cov_ratio", 0.0002)
    ub, lb = _cfg_get(pl, "clip_cov_ub", 5.0), _cfg_get(pl, "clip_cov_lb", 1.0)
    assert frac > 0, "clip_ratio should be larger than 0."
    lo, hi = _clip_bounds(config)
    lr, ratio = _ratio(old_log_prob, log_prob, clamp=False)
    a, b = -advantages * ratio, -advantages * torch.clamp(ratio, 1 - lo, 1 + hi)
    valid = response_mask > 0
    cov = (advantages - VF.masked_mean(advantages, response_mask)) * (
        log_prob - VF.masked_mean(log_prob.detach(), response_mask))
    cov = cov.detach().clone()
    cov[~valid] = -torch.inf
    cov[(b > a) & valid] = -torch.inf
    budget = max(int(frac * response_mask.sum().item()), 1)
    cand = torch.nonzero((cov < ub) & (cov > lb) & valid)
    keep = torch.ones_like(advantages)
    if len(cand) > 0:
        pick = cand[torch.randperm(len(cand))[: min(budget, len(cand))]]
        keep[pick[:, 0], pick[:, 1]] = 0
    metrics = {"actor/pg_clipfrac": VF.masked_mean((keep == 0).float(), response_mask),
               "actor/ppo_kl": VF.masked_mean(-lr, response_mask)}
    return _finish(torch.maximum(a, b) * keep, response_mask, loss_agg_mode, config, rollout_is_weights, metrics)


@register_policy_loss("kl_cov")
def compute_policy_loss_kl_cov(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                               config=None, rollout_is_weights=None):
    """KL-Cov (arXiv:2505.22617): add a KL penalty on the top-covariance fraction of tokens."""
    assert config is not None
    pl = _cfg_get(config, "policy_loss", None)
    frac = _cfg_get(pl, "kl_cov_ratio", 0.0002)
    coef = _cfg_get(pl, "ppo_kl_coef", 1.0)
    assert frac > 0, "kl_cov_ratio should be larger than 0."
    lr, ratio = _ratio(old_log_prob, log_prob, clamp=False)
    base = -advantages * ratio
    with_kl = base + coef * lr.abs()
    valid = response_mask > 0
    flat_idx = torch.nonzero(valid.reshape(-1), as_tuple=True)[0]
    losses = base
    if flat_idx.numel() > 0:
        adv_v = advantages[valid].detach().reshape(-1)
        lp_v = log_prob[valid].detach().reshape(-1)
        cov = (adv_v - adv_v.mean()) * (lp_v - lp_v.mean())
        k = max(1, int(cov.numel() * frac))
        top = flat_idx[torch.topk(cov, k, largest=True).indices]
        sel = torch.zeros(advantages.numel(), dtype=torch.bool, device=advantages.device)
        sel[top] = True
        losses = torch.where(sel.view_as(advantages), with_kl, base)
    metrics = {"actor/ppo_kl": VF.masked_mean(lr.abs(), response_mask)}
    return _finish(losses, response_mask, loss_agg_mode, config, rollout_is_weights, metrics)


@register_policy_loss("geo_mean")
def compute_policy_loss_geo_mean(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                                 config=None, rollout_is_weights=None):
    """GMPO: geometric mean of clipped token ratios per sequence."""
    assert config is not None
    lo, hi = _clip_bounds(config)
    lr = log_prob - old_log_prob
    sgn = torch.sign(advantages)
    lr_c = torch.clamp(lr, -lo, hi)
    lr_min = sgn * torch.minimum(sgn * lr, sgn * lr_c)
    n = response_mask.sum(-1)
    seq_ratio = torch.exp((lr_min * response_mask).sum(-1) / (n + 1e-8))
    seq_adv = (advantages * response_mask).sum(-1) / (n + 1e-8)
    losses = -seq_adv * seq_ratio
    if rollout_is_weights is not None:
        losses = losses * torch.exp((torch.log(rollout_is_weights + 1e-10) * response_mask).sum(-1) / (n + 1e-8))
    clipped = lr != lr_c
    metrics = {
        "actor/pg_clipfrac": VF.masked_mean((clipped & (advantages > 0)).float(), response_mask).item(),
        "actor/ppo_kl": VF.masked_mean(-lr, response_mask).item(),
        "actor/pg_clipfrac_lower": VF.masked_mean((clipped & (advantages < 0)).float(), response_mask).item(),
    }
    return losses.mean(), metrics


@register_policy_loss("dro")
def compute_policy_loss_dro(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                            config=None, rollout_is_weights=None):
    """Direct reward optimisation: log-likelihood weighted by advantage with a quadratic log-ratio penalty."""
    assert config is not None
    beta = _cfg_get(_cfg_get(config, "policy_loss", None), "dro_beta", None)
    if beta is None or beta <= 0:
        raise ValueError("policy_loss.dro_beta must be a positive value when using DRO")
    lr = log_prob - old_log_prob
    losses = -(log_prob * advantages - 0.5 * beta * lr.square())
    return _finish(losses, response_mask, loss_agg_mode, config, rollout_is_weights,
                   {"actor/ppo_kl": VF.masked_mean(-lr, response_mask)})


@register_policy_loss("cispo")
def compute_policy_loss_cispo(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                              config=None, rollout_is_weights=None):
    """CISPO: clipped, stop-gradient importance weight on the REINFORCE term."""
    assert config is not None
    lo, hi = _clip_bounds(config)
    lr, ratio = _ratio(old_log_prob, log_prob)
    w = torch.clamp(ratio, 1 - lo, 1 + hi)
    metrics = {"actor/pg_clipfrac": VF.masked_mean((ratio != w).float(), response_mask),
               "actor/ppo_kl": VF.masked_mean(-lr, response_mask), "actor/pg_clipfrac_lower": 0.0}
    return _finish(-w.detach() * advantages * log_prob, response_mask, loss_agg_mode, config, rollout_is_weights,
                   metrics)


def compute_policy_loss_reinforce(rollout_log_prob, log_prob, advantages, response_mask,
                                  loss_agg_mode="token-mean", config=None, rollout_is_weights=None):
    assert config is not None, "ActorConfig must be provided for REINFORCE loss"
    metrics = {"actor/ppo_kl": VF.masked_mean(-(log_prob - rollout_log_prob), response_mask)}
    return _finish(-advantages * log_prob, response_mask, loss_agg_mode, config, rollout_is_weights, metrics)


@register_policy_loss("bypass_mode")
def compute_policy_loss_bypass_mode(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                                    config=None, rollout_is_weights=None):
    """Bypass mode: ``old_log_prob`` IS the rollout log-prob (no separate old-policy pass); importance weights
    and rejection masks between the current policy and the rollout policy are computed on the fly."""
    from .rollout_corr_helper import compute_rollout_correction_and_rejection_mask

    assert config is not None, "config is required for bypass_mode loss"
    rc = _cfg_get(_cfg_get(config, "policy_loss", None), "rollout_correction", None)
    if rc is None:
        raise ValueError("rollout_correction config not found in policy_loss. When using loss_mode='bypass_mode', "
                         "ensure rollout_correction config is passed.")
    loss_type = _cfg_get(rc, "loss_type", "ppo_clip")
    with torch.no_grad():
        is_proto, new_mask, rc_metrics = compute_rollout_correction_and_rejection_mask(
            old_log_prob=log_prob, rollout_log_prob=old_log_prob, response_mask=response_mask,
            rollout_is=_cfg_get(rc, "rollout_is", None), rollout_is_threshold=_cfg_get(rc, "rollout_is_threshold", 2.0),
            rollout_is_batch_normalize=_cfg_get(rc, "rollout_is_batch_normalize", False),
            rollout_rs=_cfg_get(rc, "rollout_rs", None), rollout_rs_threshold=_cfg_get(rc, "rollout_rs_threshold", None))
    w = is_proto.batch["rollout_is_weights"] if is_proto is not None else None
    if loss_type == "reinforce":
        loss, metrics = compute_policy_loss_reinforce(old_log_prob, log_prob, advantages, new_mask, loss_agg_mode,
                                                      config, w)
    elif loss_type == "ppo_clip":
        loss, metrics = compute_policy_loss_vanilla(old_log_prob, log_prob, advantages, new_mask, loss_agg_mode,
                                                    config, None)
    else:
        raise ValueError(f"Invalid loss_type: {loss_type}. Must be 'reinforce' or 'ppo_clip'.")
    metrics.update(rc_metrics)
    return loss, metrics


# ----------------------------------------------------------------------------------------------- misc losses
def compute_entropy_loss(logits, response_mask, loss_agg_mode: str = "token-mean"):
    ent = VF.entropy_from_logits(logits)
    return agg_loss(loss_mat=ent, loss_mask=response_mask, loss_agg_mode=loss_agg_mode)


def compute_value_loss(vpreds, returns, values, response_mask, cliprange_value: float,
                       loss_agg_mode: str = "token-mean", dp_size: int = 1, batch_num_tokens=None,
                       global_batch_size=None, loss_scale_factor=None):
    """Clipped value loss: 0.5 * agg(max((v-R)^2, (clip(v, V_old +- c) - R)^2))."""
    vclip = VF.clip_by_value(vpreds, values - cliprange_value, values + cliprange_value)
    l1, l2 = (vpreds - returns) ** 2, (vclip - returns) ** 2
    loss = 0.5 * agg_loss(torch.max(l1, l2), response_mask, loss_agg_mode, dp_size=dp_size,
                          batch_num_tokens=batch_num_tokens, global_batch_size=global_batch_size,
                          loss_scale_factor=loss_scale_factor)
    return loss, VF.masked_mean((l2 > l1).float(), response_mask)


def kl_penalty_forward(logprob, ref_logprob, kl_penalty: str):
    d = logprob - ref_logprob
    if kl_penalty in ("kl", "k1"):
        return d
    if kl_penalty == "abs":
        return d.abs()
    if kl_penalty in ("mse", "k2"):
        return 0.5 * d.square()
    if kl_penalty in ("low_var_kl", "k3"):
        k = torch.clamp(-d, min=-20, max=20)
        return torch.clamp(torch.exp(k) - k - 1, min=-10, max=10)
    raise NotImplementedError(kl_penalty)


def kl_penalty(logprob, ref_logprob, kl_penalty: str):
    """KL estimators k1/abs/k2/k3; a trailing '+' keeps the estimator's value but uses k2's gradient."""
    base = kl_penalty[:-1] if kl_penalty.endswith("+") else kl_penalty
    fwd = kl_penalty_forward(logprob, ref_logprob, base)
    if not kl_penalty.endswith("+") or kl_penalty in ("mse", "k2"):
        return fwd
    bwd = 0.5 * (logprob - ref_logprob).square()
    return bwd - bwd.detach() + fwd.detach()


def compute_pf_ppo_reweight_data(data, reweight_method: str = "pow", weight_pow: float = 2.0):
    """PF-PPO: resample the batch with replacement according to a function of the sequence score."""
    scores = data.batch["token_level_scores"].sum(dim=-1)
    if reweight_method == "pow":
        w = scores.abs().pow(weight_pow)
    elif reweight_method == "max_min":
        w = ((scores == scores.max()) | (scores == scores.min())).float()
    elif reweight_method == "max_random":
        w = torch.where(scores == scores.max(), 0.4, 0.1)
    else:
        raise ValueError(f"Unsupported reweight_method: {reweight_method}")
    w = torch.clamp(w + 1e-8, min=1e-8)
    idx = torch.multinomial(w, scores.shape[0], replacement=True)
    out = data.select_idxs(idx)
    n = scores.shape[0]
    inp = idx.cpu().numpy()
    out.meta_info = {k: ([v[i] for i in inp] if isinstance(v, list) and len(v) == n else v)
                     for k, v in data.meta_info.items()}
    return out
