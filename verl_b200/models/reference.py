"""Plain-PyTorch (autograd) restatement of the decoder, used as the numerical oracle in tests.

It consumes the same fused parameter views as :class:`DecoderModel` but is written with ordinary torch
ops, one sequence at a time, so its gradients come from autograd rather than from the hand-written
backward pass.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as TF

from .config import ModelConfig

__all__ = ["reference_hidden", "reference_logprobs", "reference_values"]


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def _rope(x, pos, theta):
    hd = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    ang = pos.double().unsqueeze(-1) * inv
    c, s = ang.cos().float().unsqueeze(1), ang.sin().float().unsqueeze(1)
    a, b = x[..., : hd // 2].float(), x[..., hd // 2 :].float()
    return torch.cat([a * c - b * s, b * c + a * s], -1).to(x.dtype)


def reference_hidden(cfg: ModelConfig, P: dict, input_ids: torch.Tensor, lengths: list[int]) -> torch.Tensor:
    """Final-norm hidden states [T, H] for packed ``input_ids`` with the given sequence lengths."""
    outs = []
    s0 = 0
    nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    for n in lengths:
        ids = input_ids[s0 : s0 + n]
        s0 += n
        pos = torch.arange(n)
        x = TF.embedding(ids, P["embed_tokens.weight"])
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            h = _rms(x, P[p + "input_layernorm.weight"], cfg.rms_norm_eps)
            qkv = TF.linear(h, P[p + "self_attn.qkv_proj.weight"], P.get(p + "self_attn.qkv_proj.bias"))
            q = qkv[:, : cfg.q_size].reshape(n, nh, hd)
            k = qkv[:, cfg.q_size : cfg.q_size + cfg.kv_size].reshape(n, nkv, hd)
            v = qkv[:, cfg.q_size + cfg.kv_size :].reshape(n, nkv, hd)
            if cfg.qk_norm:
                q = _rms(q, P[p + "self_attn.q_norm.weight"], cfg.rms_norm_eps)
                k = _rms(k, P[p + "self_attn.k_norm.weight"], cfg.rms_norm_eps)
            q, k = _rope(q, pos, cfg.rope_theta), _rope(k, pos, cfg.rope_theta)
            g = nh // nkv
            kk, vv = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
            sc = torch.einsum("qhd,khd->hqk", q.float(), kk.float()) / math.sqrt(hd)
            mask = torch.ones(n, n, dtype=torch.bool).tril()
            sc = sc.masked_fill(~mask, float("-inf"))
            att = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), vv.float()).to(x.dtype).reshape(n, nh * hd)
            x = x + TF.linear(att, P[p + "self_attn.o_proj.weight"])
            h = _rms(x, P[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
            if cfg.is_moe:
                probs = torch.softmax(TF.linear(h, P[p + "mlp.gate.weight"]).float(), -1)
                w, idx = torch.topk(probs, cfg.num_experts_per_tok, -1)
                if cfg.norm_topk_prob:
                    w = w / w.sum(-1, keepdim=True)
                y = torch.zeros_like(h, dtype=torch.float32)
                for e in range(cfg.num_experts):
                    sel = idx == e
                    if not sel.any():
                        continue
                    tok = sel.any(-1)
                    gu = TF.linear(h[tok], P[p + "mlp.experts.gate_up_proj"][e])
                    g_, u_ = gu.chunk(2, -1)
                    ye = TF.linear(TF.silu(g_) * u_, P[p + "mlp.experts.down_proj"][e])
                    y[tok] += ye.float() * (w * sel)[tok].sum(-1, keepdim=True)
                x = x + y.to(x.dtype)
            else:
                gu = TF.linear(h, P[p + "mlp.gate_up_proj.weight"])
                g_, u_ = gu.chunk(2, -1)
                x = x + TF.linear(TF.silu(g_) * u_, P[p + "mlp.down_proj.weight"])
        outs.append(_rms(x, P["norm.weight"], cfg.rms_norm_eps))
    return torch.cat(outs, 0)


def reference_logprobs(cfg, P, input_ids, lengths, labels, temperature: float = 1.0):
    h = reference_hidden(cfg, P, input_ids, lengths)
    head = P.get("lm_head.weight", P["embed_tokens.weight"])
    logits = TF.linear(h, head).float() / max(temperature, 1e-8)
    lse = torch.logsumexp(logits, -1)
    lp = logits.gather(-1, labels.unsqueeze(-1)).squeeze(-1) - lse
    ent = lse - (torch.softmax(logits, -1) * logits).sum(-1)
    return lp, ent


def reference_values(cfg, P, input_ids, lengths):
    h = reference_hidden(cfg, P, input_ids, lengths)
    return TF.linear(h, P["v_head.weight"])[:, 0].float()
