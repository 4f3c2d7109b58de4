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


def _causal_pairs(s: int, window: int = 0) -> float:
    """Number of (query, key) pairs a causal layer evaluates for a sequence of ``s`` tokens; ``window`` > 0 limits every
    query to its ``window`` most recent keys."""
    if window <= 0 or s <= window:
        return s * (s + 1) / 2.0
    return window * (window + 1) / 2.0 + (s - window) * float(window)


def _terms_from_hf(d: dict) -> tuple[float, list[tuple[int, int, float]]]:
    """(multiply-accumulates per token in the projections, MLPs, routers and LM head; attention layer classes as
    ``(layers, window, heads * (score width + value width))``) of a library configuration. Covers latent attention with
    dense-then-sparse stacks (DeepSeek-V2/V3), sliding / full layer patterns (GPT-OSS, Gemma-2/3, Mistral) and plain
    grouped-query decoders; unknown fields fall back to the dense decoder reading of the configuration."""
    t = d.get("text_config") if isinstance(d.get("text_config"), dict) else d
    h, L, H = t["hidden_size"], t["num_hidden_layers"], t["num_attention_heads"]
    kvh = t.get("num_key_value_heads") or H
    if t.get("kv_lora_rank"):                                   # multi-head latent attention
        nope, rope, vd, r = t["qk_nope_head_dim"], t["qk_rope_head_dim"], t["v_head_dim"], t["kv_lora_rank"]
        qr = t.get("q_lora_rank") or 0
        q = (h * qr + qr * H * (nope + rope)) if qr else h * H * (nope + rope)
        attn_lin = q + h * (r + rope) + r * H * (nope + vd) + H * vd * h
        width = H * (nope + rope + vd)
    else:
        hd = t.get("head_dim") or h // H
        attn_lin = h * (H + 2 * kvh) * hd + H * hd * h
        width = H * 2 * hd
    experts = t.get("n_routed_experts") or t.get("num_local_experts") or t.get("num_experts") or 0
    if experts:
        top_k = t.get("num_experts_per_tok", 1)
        ie = t.get("moe_intermediate_size") or t.get("intermediate_size")
        shared = (t.get("n_shared_experts") or 0) * ie + (t.get("shared_expert_intermediate_size") or 0)
        sparse = 3 * h * (ie * top_k + shared) + h * experts
        n_dense = min(L, t.get("first_k_dense_replace") or 0)
        mlp_total = n_dense * 3 * h * t.get("intermediate_size", ie) + (L - n_dense) * sparse
    else:
        mlp_total = L * 3 * h * t["intermediate_size"]
    linear = L * attn_lin + mlp_total + t["vocab_size"] * h
    window = int(t.get("sliding_window") or 0)
    kinds = t.get("layer_types")
    if kinds and window:
        n_slide = sum(1 for k in kinds[:L] if "sliding" in str(k))
    elif window and t.get("sliding_window_pattern"):           # every n-th layer is global
        n_slide = L - L // int(t["sliding_window_pattern"])
    elif window and t.get("model_type") in ("mistral", "gemma2"):
        n_slide = L if t.get("model_type") == "mistral" else L // 2
    else:
        n_slide = 0
    classes = [(L - n_slide, 0, float(width))] + ([(n_slide, window, float(width))] if n_slide else [])
    return float(linear), classes


class FlopsCounter:
    """Training FLOPs (forward + backward = 3x forward) of one batch of sequences. Natively supported families are read
    from the architecture description; any other family from its library configuration (``_terms_from_hf``)."""

    def __init__(self, config):
        self.config = config
        self._generic = None
        if getattr(config, "is_generic", False):
            try:
                self._generic = _terms_from_hf(config.extra["hf_config"])
            except (KeyError, TypeError):
                self._generic = None

    def _dense_per_token(self) -> float:
        if self._generic is not None:
            return self._generic[0]
        c = self.config
        h = c.hidden_size
        attn_lin = h * (c.q_size + 2 * c.kv_size) + c.q_size * h
        if getattr(c, "is_moe", False) and c.is_moe:
            mlp = 3 * h * c.moe_intermediate_size * c.num_experts_per_tok + h * c.num_experts
            if getattr(c, "shared_expert_intermediate_size", 0):
                mlp += 3 * h * c.shared_expert_intermediate_size + h
        else:
            mlp = 3 * h * c.intermediate_size
        emb = c.vocab_size * h  # LM head (the embedding gather is free)
        return (attn_lin + mlp) * c.num_hidden_layers + emb

    def _attention_forward_flops(self, batch_seqlens: Sequence[int]) -> float:
        """QK^T and PV of the causal layers: 2 FLOPs per multiply-accumulate, (score + value width) per pair."""
        if self._generic is not None:
            return sum(2.0 * n * width * sum(_causal_pairs(int(s), w) for s in batch_seqlens) for n, w, width in self._generic[1])
        c = self.config
        sq = float(sum(int(s) ** 2 for s in batch_seqlens))
        return 4.0 * sq * c.head_dim * c.num_attention_heads * c.num_hidden_layers / 2.0

    def estimate_flops(self, batch_seqlens: Sequence[int], delta_time: float):
        """Returns (achieved TFLOPS, promised TFLOPS). ``batch_seqlens``: valid tokens per sequence."""
        total = 3.0 * self.forward_flops(batch_seqlens)
        return total / max(delta_time, 1e-9) / 1e12, get_device_flops("T")

    def forward_flops(self, batch_seqlens: Sequence[int]) -> float:
        tokens = float(sum(batch_seqlens))
        return 2.0 * self._dense_per_token() * tokens + self._attention_forward_flops(batch_seqlens)
