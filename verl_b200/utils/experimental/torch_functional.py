"""``FusedLinearForPPO``: module-style wrapper (``forward(hidden, weight, input_ids, temperature) -> (log_probs,
entropy)``) of the fused hidden -> log-prob / entropy head, for [batch, seq, hidden] inputs.

Parity target: ``verl/utils/experimental/torch_functional.py:27-231`` (chunked pure-torch formulation; here the chunks
are the vocabulary chunks of the fused kernels, the [tokens, vocabulary] logits are never formed).
"""

from __future__ import annotations

import torch

from ..kernel.linear_cross_entropy import linear_cross_entropy

__all__ = ["FusedLinearForPPO"]


class FusedLinearForPPO(torch.nn.Module):
    def __init__(self, chunk_size: int = 512):
        super().__init__()
        self.chunk_size = chunk_size  # kept for interface parity; the kernels tile internally

    def forward(self, hidden_states: torch.Tensor, vocab_weights: torch.Tensor, input_ids: torch.Tensor, temperature: float = 1.0):
        """``input_ids`` are the labels aligned with ``hidden_states`` (already shifted by the caller)."""
        squeeze = hidden_states.dim() == 2
        h = hidden_states.unsqueeze(0) if squeeze else hidden_states
        ids = input_ids.unsqueeze(0) if squeeze else input_ids
        lp, ent = linear_cross_entropy(h, vocab_weights, ids, temperature, "none")
        return (lp.squeeze(0), ent.squeeze(0)) if squeeze else (lp, ent)
