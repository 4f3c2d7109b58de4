"""Distillation losses when the student's vocabulary is split over a tensor-parallel group: every rank holds the logits
(or the head rows) of one vocabulary slice, the log-softmax normaliser and the top-k gather are completed with two small
all-reduces, and the backward pass needs no communication.

Parity target: ``verl/trainer/distillation/megatron/losses.py`` (``vocab_parallel_log_softmax`` :27,
``_VocabParallelKLDivergence`` :58, ``compute_forward_kl_topk`` :264).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

__all__ = ["vocab_parallel_log_softmax", "vocab_parallel_topk_log_probs", "compute_forward_kl_topk_vocab_parallel"]


class _AllReduceSum(torch.autograd.Function):
    """Sum over the group in forward; the gradient of a sum is the incoming gradient on every rank."""

    @staticmethod
    def forward(ctx, x, group):
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _AllReduceSumPartialUse(torch.autograd.Function):
    """Sum over the group whose result every rank uses for a different part of the (replicated) loss: the complete
    gradient of the sum is the sum of the ranks' partial gradients, so the backward pass reduces as well."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def vocab_parallel_log_softmax(local_logits: torch.Tensor, group) -> torch.Tensor:
    """``log_softmax`` over the full vocabulary for this rank's slice [..., V_local] of the logits."""
    x = local_logits.float()
    m = x.detach().amax(-1, keepdim=True)
    dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
    # each rank reads the normaliser only for the entries of its own slice
    se = _AllReduceSumPartialUse.apply(torch.exp(x - m).sum(-1, keepdim=True), group)
    return x - m - torch.log(se)


def vocab_parallel_topk_log_probs(local_log_probs: torch.Tensor, ids: torch.Tensor, vocab_start: int, group) -> torch.Tensor:
    """Full-vocabulary log-probs of ``ids`` [..., k] gathered from the slices: each id lives on exactly one rank."""
    Vl = local_log_probs.shape[-1]
    loc = ids - vocab_start
    mine = (loc >= 0) & (loc < Vl)
    got = torch.gather(local_log_probs, -1, loc.clamp(0, Vl - 1)) * mine
    return _AllReduceSum.apply(got, group)


def compute_forward_kl_topk_vocab_parallel(local_student_logits: torch.Tensor, teacher_topk_log_probs: torch.Tensor,
                                           teacher_topk_ids: torch.Tensor, vocab_start: int, group, clamp: float = -10.0):
    """Forward KL(teacher || student) restricted to the teacher's top-k tokens, both renormalised over those k tokens.
    Returns (per-position loss, student mass on the top-k, teacher mass on the top-k)."""
    logp = vocab_parallel_log_softmax(local_student_logits, group)
    s = vocab_parallel_topk_log_probs(logp, teacher_topk_ids, vocab_start, group).clamp(min=clamp)
    t = teacher_topk_log_probs.float().clamp(min=clamp)
    s_mass, t_mass = s.exp().sum(-1), t.exp().sum(-1)
    s_n = s - torch.logsumexp(s, -1, keepdim=True)
    t_n = t - torch.logsumexp(t, -1, keepdim=True)
    return (t_n.exp() * (t_n - s_n)).sum(-1), s_mass.detach(), t_mass
