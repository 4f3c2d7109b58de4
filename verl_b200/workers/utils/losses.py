"""Worker-side loss functions: SFT, PPO actor objective, critic value loss.

Each takes ``(config, model_output, data, dp_group)`` and returns ``(loss, metrics)`` where ``loss`` is scaled
so that the data-parallel gradient mean equals the gradient of the global-batch objective.

Parity target: ``verl/workers/utils/losses.py`` (``sft_loss`` :28-54, ``ppo_loss`` :57-144, ``value_loss`` :147-205).
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from ...trainer.ppo.core_algos import agg_loss, compute_value_loss, get_policy_loss_fn, kl_penalty
from ...utils import torch_functional as VF

__all__ = ["sft_loss", "ppo_loss", "value_loss"]


def _g(cfg, key, default=None):
    if cfg is None:
        return default
    v = cfg.get(key, default) if hasattr(cfg, "get") else getattr(cfg, key, default)
    return default if v is None else v


def _info(data) -> dict:
    info = data.get("global_batch_info", None) if hasattr(data, "get") else None
    info = dict(info or {})
    return {k: info.get(k) for k in ("dp_size", "batch_num_tokens", "global_batch_size", "loss_scale_factor")
            if info.get(k) is not None}


def sft_loss(config, model_output: dict, data, dp_group=None):
    """Negative log-likelihood on the response tokens, global token mean."""
    lp = model_output["log_probs"]
    mask = data["response_mask"].to(lp.dtype) if "response_mask" in data else data["loss_mask"].to(lp.dtype)
    loss = agg_loss(-lp, mask, "token-mean", **{k: v for k, v in _info(data).items() if k in ("dp_size", "batch_num_tokens")})
    return loss, {"sft/loss": loss.detach().item()}


class _CfgView(dict):
    """ActorConfig fields + per-call ``global_batch_info`` presented through ``.get``/attribute access."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError:
            raise AttributeError(k) from None


def ppo_loss(config, model_output: dict, data, dp_group=None):
    """``pg_loss - entropy_coeff * entropy + kl_loss_coef * KL(pi || ref)`` with the configured policy loss."""
    lp = model_output["log_probs"]
    mask = data["response_mask"].to(lp.dtype)
    old = data["old_log_probs"] if "old_log_probs" in data else lp.detach()
    adv = data["advantages"]
    info = _info(data)
    view = _CfgView({k: _g(config, k) for k in ("clip_ratio", "clip_ratio_low", "clip_ratio_high", "clip_ratio_c",
                                                "tau_pos", "tau_neg", "policy_loss")})
    view["global_batch_info"] = info
    mode = _g(_g(config, "policy_loss", None), "loss_mode", "vanilla")
    agg = _g(config, "loss_agg_mode", "token-mean")
    is_w = data["rollout_is_weights"] if "rollout_is_weights" in data else None
    pg_loss, metrics = get_policy_loss_fn(mode)(old_log_prob=old, log_prob=lp, advantages=adv, response_mask=mask,
                                                loss_agg_mode=agg, config=view, rollout_is_weights=is_w)
    loss = pg_loss
    metrics = dict(metrics)
    metrics["actor/pg_loss"] = pg_loss.detach().item()
    ec = float(_g(config, "entropy_coeff", 0.0) or 0.0)
    if "entropy" in model_output and model_output["entropy"] is not None:
        ent = agg_loss(model_output["entropy"], mask, agg, **info)
        metrics["actor/entropy"] = ent.detach().item()
        if ec != 0.0:
            loss = loss - ec * ent
    if _g(config, "use_kl_loss", False) and "ref_log_prob" in data:
        kld = kl_penalty(lp, data["ref_log_prob"], _g(config, "kl_loss_type", "low_var_kl"))
        kl = agg_loss(kld, mask, agg, **info)
        loss = loss + float(_g(config, "kl_loss_coef", 0.001)) * kl
        metrics["actor/kl_loss"] = kl.detach().item()
        metrics["actor/kl_coef"] = float(_g(config, "kl_loss_coef", 0.001))
    return loss, metrics


def value_loss(config, model_output: dict, data, dp_group=None):
    """Clipped value regression against the returns."""
    v = model_output["values"]
    mask = data["response_mask"].to(v.dtype)
    info = _info(data)
    loss, clipfrac = compute_value_loss(vpreds=v, returns=data["returns"], values=data["values"], response_mask=mask,
                                        cliprange_value=float(_g(config, "cliprange_value", 0.5)),
                                        loss_agg_mode=_g(config, "loss_agg_mode", "token-mean"), **info)
    return loss, {"critic/vf_loss": loss.detach().item(), "critic/vf_clipfrac": clipfrac.detach().item(),
                  "critic/vpred_mean": VF.masked_mean(v, mask).detach().item()}
