"""Autograd entry point of the fused LM head: ``(hidden, weight, labels) -> (log-probs, entropy)`` without ever forming the
[tokens, vocabulary] logits, differentiable with respect to ``hidden`` and ``weight``. On a GPU the forward is the tcgen05
GEMM with the online-softmax epilogue and the backward the chunked d_logits kernel feeding two tensor-core GEMMs; on the
host the same math runs in fp32. With ``dist_process_group`` the vocabulary is split over the group (each rank passes its
rows of ``weight``).

For model code written against autograd; the decoder's hand-scheduled backward calls the same kernels directly.
Parity target: ``verl/utils/kernel/linear_cross_entropy.py:38-119`` (``LinearCrossEntropy``), ``kernels.py`` (K1-K6).
"""

from __future__ import annotations

from typing import Optional

import torch

from ...ops import functional as F

__all__ = ["LinearCrossEntropy", "linear_cross_entropy"]


class LinearCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                reduction: str = "none", dist_process_group=None, vocab_start: int = 0):
        assert reduction in ("none", "sum", "mean")
        shape = labels.shape
        h2, l1 = hidden.reshape(-1, hidden.shape[-1]).contiguous(), labels.reshape(-1).contiguous()
        if dist_process_group is not None:
            lp, ent, lse = F.lmhead_logprob_entropy_vocab_parallel(h2, weight, l1, temperature, vocab_start, dist_process_group)
        else:
            lp, ent, lse = F.lmhead_logprob_entropy(h2, weight, l1, temperature)
        ctx.save_for_backward(h2, weight, l1, lse, ent)
        ctx.meta = (float(temperature), reduction, dist_process_group, int(vocab_start), hidden.shape, shape)
        if reduction == "sum":
            return lp.sum(), ent.sum()
        if reduction == "mean":
            return lp.mean(), ent.mean()
        return lp.view(shape), ent.view(shape)

    @staticmethod
    def backward(ctx, g_lp: Optional[torch.Tensor], g_ent: Optional[torch.Tensor]):
        h2, weight, l1, lse, ent = ctx.saved_tensors
        temperature, reduction, group, vocab_start, h_shape, shape = ctx.meta
        n = l1.numel()

        def expand(g):
            if g is None:
                return None
            if reduction == "none":
                return g.reshape(-1).float().contiguous()
            return (g.float() / (n if reduction == "mean" else 1)).expand(n).contiguous()

        g_lp, g_ent = expand(g_lp), expand(g_ent)
        if g_lp is None:
            g_lp = torch.zeros(n, dtype=torch.float32, device=h2.device)
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device) if ctx.needs_input_grad[1] else None
        dh = F.lmhead_backward(h2, weight, l1, temperature, lse, ent, g_lp, g_ent, dw, vocab_start=vocab_start)
        if group is not None:
            import torch.distributed as dist

            dh = dh.float()
            dist.all_reduce(dh, group=group)
        return (dh.to(h2.dtype).view(h_shape) if ctx.needs_input_grad[0] else None, dw.to(weight.dtype) if dw is not None else None,
                None, None, None, None, None)


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                         reduction: str = "none", dist_process_group=None, vocab_start: int = 0):
    """(log_probs, entropy) of ``labels`` under ``softmax(hidden @ weight^T / temperature)``."""
    return LinearCrossEntropy.apply(hidden, weight, labels, temperature, reduction, dist_process_group, vocab_start)
