"""On-policy distillation losses: the student is trained on its own samples towards a teacher's distribution.

* ``forward_kl_topk`` - the teacher supplies, per response token, its top-k token ids and log-probs; the loss is
  ``sum_k p_t(k) * (log p_t(k) - log q_s(k))`` over that support, optionally plus a tail term that matches the
  probability mass outside the support.
* ``reverse_kl_k1/k2/k3`` (aliases ``k1``, ``abs``, ``mse``, ``low_var_kl`` ...) - single-sample estimators of
  KL(student || teacher) from the log-probs of the sampled token under both models.

Per-token losses are clamped to ``loss_max_clamp`` and reduced with the actor's ``loss_agg_mode``; with
``use_policy_gradient`` the negated, detached per-token loss is used as an advantage in a PPO-style clipped objective
instead of being differentiated directly.

Parity target: ``verl/trainer/distillation/losses.py`` (registry :46-106, ``compute_topk_loss`` :123,
``distillation_ppo_loss`` :165, ``distillation_loss`` :230-300, ``compute_forward_kl_topk`` :305,
reverse-KL estimators :370-405) and ``verl/trainer/distillation/fsdp/losses.py:26-149``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch

from ...base_config import BaseConfig
from ..ppo.core_algos import agg_loss, get_policy_loss_fn, kl_penalty

__all__ = ["DistillationLossConfig", "DistillationConfig", "DistillationLossSettings", "register_distillation_loss",
           "get_distillation_loss_fn", "get_distillation_loss_settings", "is_distillation_enabled", "distillation_loss",
           "compute_forward_kl_topk", "student_topk_log_probs", "kl_divergence", "distillation_ppo_loss"]


@dataclass
class DistillationLossConfig(BaseConfig):
    loss_mode: str = "k3"              # k1 | k2 | k3 | abs | mse | low_var_kl (sampled-token estimators) | forward_kl_topk
    topk: int = 32
    use_task_rewards: bool = True      # False: the task's policy-gradient loss is dropped, distillation alone trains the student
    distillation_loss_coef: float = 1.0  # weight of the distillation term beside the task loss
    use_tail_term: bool = False        # add the KL term of the mass outside the top-k support
    log_prob_min_clamp: Optional[float] = -10.0
    loss_max_clamp: Optional[float] = 10.0
    use_policy_gradient: bool = False
    policy_loss_mode: str = "vanilla"
    clip_ratio: float = 0.2
    clip_ratio_low: float = 0.2
    clip_ratio_high: float = 0.2
    clip_ratio_c: float = 3.0
    loss_coef: float = 1.0
    global_batch_info: dict = field(default_factory=dict)


@dataclass
class DistillationConfig(BaseConfig):
    enabled: bool = False
    num_teachers: int = 1
    teacher_key: str = "data_source"   # non-tensor field that routes a sample to one of several teachers
    # name -> {key: value of teacher_key served by this teacher (null = default), model_path, num_replicas}
    teacher_models: dict = field(default_factory=dict)
    n_gpus_per_node: int = 8
    nnodes: int = 0                    # 0: the teachers share the trainer's GPUs
    distillation_loss: DistillationLossConfig = field(default_factory=DistillationLossConfig)


@dataclass
class DistillationLossSettings:
    names: list
    use_topk: bool = False             # needs teacher_ids / teacher_logprobs [b, R, k]
    use_estimator: bool = False        # needs teacher log-prob of the sampled token [b, R]

    def __post_init__(self):
        self.names = [self.names] if isinstance(self.names, str) else list(self.names)


DistillationLossFn = Callable[..., tuple[torch.Tensor, dict]]
_LOSSES: dict[str, DistillationLossFn] = {}
_SETTINGS: dict[str, DistillationLossSettings] = {}


def register_distillation_loss(settings: DistillationLossSettings):
    def deco(fn):
        for n in settings.names:
            if n in _LOSSES:
                raise ValueError(f"Distillation loss function with name '{n}' is already registered.")
            _LOSSES[n], _SETTINGS[n] = fn, settings
        return fn

    return deco


def get_distillation_loss_fn(name: str) -> DistillationLossFn:
    if name not in _LOSSES:
        raise ValueError(f"Unsupported distillation loss: {name} (known: {sorted(_LOSSES)})")
    return _LOSSES[name]


def get_distillation_loss_settings(name: str) -> DistillationLossSettings:
    get_distillation_loss_fn(name)
    return _SETTINGS[name]


def is_distillation_enabled(config: Optional[DistillationConfig]) -> bool:
    return bool(config is not None and (config.get("enabled", False) if hasattr(config, "get") else config.enabled))


def kl_divergence(log_q: torch.Tensor, log_p: torch.Tensor) -> torch.Tensor:
    """KL(p || q) summed over the last dimension, from log-probabilities."""
    p = log_p.exp()
    return (p * (log_p - log_q)).sum(-1)


def student_topk_log_probs(hidden: torch.Tensor, weight: torch.Tensor, ids: torch.Tensor, lse: Optional[torch.Tensor] = None,
                           chunk: int = 2048) -> torch.Tensor:
    """``log q_s(ids)`` [T, k] from final hidden states [T, H] and the LM-head weight [V, H] without materialising
    [T, V] logits when ``lse`` [T] is given (else the log-sum-exp is computed chunk by chunk)."""
    out = []
    for lo in range(0, hidden.size(0), chunk):
        h = hidden[lo : lo + chunk]
        w = weight[ids[lo : lo + chunk]]                      # [t, k, H]
        z = torch.einsum("th,tkh->tk", h.float(), w.float())
        l = lse[lo : lo + chunk] if lse is not None else torch.logsumexp(h.float() @ weight.float().t(), -1)
        out.append(z - l[:, None])
    return torch.cat(out, 0)


def compute_forward_kl_topk(student_logits: Optional[torch.Tensor], teacher_topk_log_probs: torch.Tensor, teacher_topk_ids: torch.Tensor,
                            config: DistillationLossConfig, student_topk_logp: Optional[torch.Tensor] = None) -> dict:
    """Per-token forward KL on the teacher's support. Give either full ``student_logits`` [..., V] or the already
    gathered ``student_topk_logp`` [..., k]. Returns ``distillation_losses``, ``student_mass``, ``teacher_mass``."""
    if student_topk_logp is None:
        student_topk_logp = torch.log_softmax(student_logits.float(), -1).gather(-1, teacher_topk_ids)
    lp_t = teacher_topk_log_probs.float()
    lq_s = student_topk_logp.float()
    if config.log_prob_min_clamp is not None:
        lq_s = lq_s.clamp_min(config.log_prob_min_clamp)
        lp_t = lp_t.clamp_min(config.log_prob_min_clamp)
    loss = kl_divergence(lq_s, lp_t)
    t_mass, s_mass = lp_t.exp().sum(-1), lq_s.exp().sum(-1)
    if config.use_tail_term:
        eps = 1e-6
        tt, ts = (1 - t_mass).clamp(eps, 1.0), (1 - s_mass).clamp(eps, 1.0)
        loss = loss + tt * (tt.log() - ts.log())
    return {"distillation_losses": loss, "student_mass": s_mass, "teacher_mass": t_mass}


@register_distillation_loss(DistillationLossSettings(names=["forward_kl_topk"], use_topk=True))
def _forward_kl_topk(config, distillation_config, model_output: dict, data: dict):
    lc = distillation_config.distillation_loss
    out = compute_forward_kl_topk(model_output.get("logits"), data["teacher_logprobs"], data["teacher_ids"], lc,
                                  student_topk_logp=model_output.get("topk_log_probs"))
    m = data["response_mask"].bool()
    metrics = {"distillation/student_mass": out["student_mass"][m].mean().item(), "distillation/teacher_mass": out["teacher_mass"][m].mean().item()}
    return out["distillation_losses"], metrics


@register_distillation_loss(DistillationLossSettings(
    names=["k1", "kl", "abs", "k2", "mse", "k3", "low_var_kl", "reverse_kl_k1", "reverse_kl_k2", "reverse_kl_k3"], use_estimator=True))
def _reverse_kl_estimator(config, distillation_config, model_output: dict, data: dict):
    mode = distillation_config.distillation_loss.loss_mode.replace("reverse_kl_", "")
    logp_s = model_output["log_probs"]
    logp_t = data["teacher_logprobs"]
    if logp_t.dim() == logp_s.dim() + 1:  # top-1 of a top-k record
        logp_t = logp_t[..., 0]
    loss = kl_penalty(logp_s, logp_t, mode)
    m = data["response_mask"].bool()
    return loss, {"distillation/teacher_logprob": logp_t[m].mean().item()}


def distillation_ppo_loss(config, distillation_config: DistillationConfig, model_output: dict, data: dict, dp_group=None):
    """The actor's loss under on-policy distillation: task (PPO / GRPO) loss and distillation term combined.

    * ``use_task_rewards`` and ``use_policy_gradient`` both off: only the distillation term (the policy loss is not even
      computed);
    * ``use_task_rewards`` off, ``use_policy_gradient`` on: the policy loss is computed for its metrics and dropped, the
      distillation term (itself a policy-gradient loss with ``-distillation loss`` as advantage) has weight 1;
    * ``use_task_rewards`` on: ``task loss + distillation_loss_coef * distillation term``.

    Parity target: ``verl/trainer/distillation/losses.py:165-227``."""
    from ...workers.utils.losses import ppo_loss

    lc = distillation_config.distillation_loss
    d_loss, d_metrics = distillation_loss(config, distillation_config, model_output, data)
    if not lc.use_task_rewards and not lc.use_policy_gradient:
        loss, metrics = 0.0, {}
    else:
        loss, metrics = ppo_loss(config, model_output, data, dp_group)
        if not lc.use_task_rewards:
            loss = 0.0
    metrics = dict(metrics)
    metrics.update(d_metrics)
    coef = float(lc.distillation_loss_coef) if lc.use_task_rewards else 1.0
    return loss + d_loss * coef, metrics


def distillation_loss(config, distillation_config: DistillationConfig, model_output: dict, data: dict) -> tuple[torch.Tensor, dict[str, Any]]:
    """Scalar loss and metrics; ``config`` is the actor config (``loss_agg_mode``, global batch info)."""
    lc = distillation_config.distillation_loss
    losses, metrics = get_distillation_loss_fn(lc.loss_mode)(config=config, distillation_config=distillation_config,
                                                             model_output=model_output, data=data)
    mask = data["response_mask"]
    sel = losses[mask.bool()]
    if sel.numel():
        metrics.update({"distillation/loss_min": sel.min().item(), "distillation/loss_max": sel.max().item()})
    if lc.loss_max_clamp is not None:
        losses = losses.clamp(min=-lc.loss_max_clamp, max=lc.loss_max_clamp)
    g = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
    info = dict(data.get("global_batch_info") or g("global_batch_info", {}) or {})
    agg_mode = g("loss_agg_mode", "token-mean")
    if lc.use_policy_gradient:
        fn = get_policy_loss_fn(lc.policy_loss_mode)
        lc.global_batch_info.update(info)
        loss, pg = fn(old_log_prob=data["old_log_probs"], log_prob=model_output["log_probs"], advantages=-losses.detach(),
                      response_mask=mask, loss_agg_mode=agg_mode, config=lc, rollout_is_weights=data.get("rollout_is_weights"))
        metrics.update({f"distillation/{k[len('actor/'):] if k.startswith('actor/') else k}": v for k, v in pg.items()})
    else:
        loss = agg_loss(loss_mat=losses, loss_mask=mask, loss_agg_mode=agg_mode, **info)
    metrics["distillation/loss"] = float(loss.detach())
    return loss * lc.loss_coef, metrics
