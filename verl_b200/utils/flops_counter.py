"""Model FLOPs estimation and device peak table for MFU reporting.

Parity target: ``verl/utils/flops_counter.py`` (peak table :22-45, per-architecture estimators :92-746).
Dense peak numbers are the marketing bf16 figures the reference assumes; the measured cuBLAS throughput of a
particular machine can be supplied through ``VERL_DEVICE_PEAK_TFLOPS``.
"""

from __future__ import annotations

import os
from typing import Sequence

import torch

__all__ = ["get_device_flops", "FlopsCounter", "DEVICE_PEAK_FLOPS"]

DEVICE_PEAK_FLOPS = {
    "GB200": 2.5e15, "B200": 2.25e15, "B300": 2.25e15, "H200": 989e12, "H100": 989e12, "H800": 989e12, "H20": 148e12,
    "A100": 312e12, "A800": 312e12, "L40S": 362e12, "L40": 181e12, "L20": 119.5e12, "A6000": 38.7e12, "4090": 165e12,
    "MI300X": 1336e12, "910B": 354e12, "CPU": 448e9,
}


def get_device_flops(unit: str = "T") -> float:
    env = os.getenv("VERL_DEVICE_PEAK_TFLOPS")
    if env:
        flops = float(env) * 1e12
    else:
        name = torch.cuda.get_device_name() if torch.cuda.is_available() else "CPU"
        flops = float("inf")
        for key, val in DEVICE_PEAK_FLOPS.items():
            if key in name:
                flops = val
                break
    div = {"B": 1e9, "K": 1e3, "M": 1e6, "G": 1e9, "T": 1e12, "P": 1e15}[unit]
    return flops / div


class FlopsCounter:
    """Training FLOPs (forward + backward = 3x forward) of one batch of sequences for the supported families."""

    def __init__(self, config):
        self.config = config

    def _dense_per_token(self) -> float:
        c = self.config
        h = c.hidden_size
        attn_lin = h * (c.q_size + 2 * c.kv_size) + c.q_size * h
        if getattr(c, "is_moe", False) and c.is_moe:
            mlp = 3 * h * c.moe_intermediate_size * c.num_experts_per_tok + h * c.num_experts
        else:
            mlp = 3 * h * c.intermediate_size
        emb = c.vocab_size * h  # LM head (the embedding gather is free)
        return (attn_lin + mlp) * c.num_hidden_layers + emb

    def estimate_flops(self, batch_seqlens: Sequence[int], delta_time: float):
        """Returns (achieved TFLOPS, promised TFLOPS). ``batch_seqlens``: valid tokens per sequence."""
        c = self.config
        tokens = float(sum(batch_seqlens))
        dense = 6.0 * self._dense_per_token() * tokens
        sq = float(sum(int(s) ** 2 for s in batch_seqlens))
        attn = 12.0 * sq * c.head_dim * c.num_attention_heads * c.num_hidden_layers / 2.0  # causal
        achieved = (dense + attn) / max(delta_time, 1e-9) / 1e12
        return achieved, get_device_flops("T")

    def forward_flops(self, batch_seqlens: Sequence[int]) -> float:
        c = self.config
        tokens = float(sum(batch_seqlens))
        sq = float(sum(int(s) ** 2 for s in batch_seqlens))
        return 2.0 * self._dense_per_token() * tokens + 4.0 * sq * c.head_dim * c.num_attention_heads * c.num_hidden_layers / 2.0
