"""Functional front-end of the native kernels.

Every function dispatches on the device of its input: CUDA tensors go to the hand-written sm_100a
kernels (bf16 activations, fp32 statistics); CPU tensors take a plain PyTorch path that doubles as the
fp32 oracle in the tests.  Nothing here silently falls back on a GPU: a missing native library raises.

Weight gradients follow the "main_grad" convention: when a parameter carries an fp32 ``main_grad``
buffer, backward GEMMs accumulate straight into it (tcgen05 wgrad with a read-modify-write epilogue) and
autograd sees ``None`` for that parameter.
"""

from __future__ import annotations

import math
from typing import Optional

import os

import torch
import torch.nn.functional as F

from . import audit, native

__all__ = [
    "gemm",
    "linear",
    "rms_norm",
    "rms_norm_bwd",
    "rope_table",
    "apply_rope_",
    "swiglu",
    "swiglu_bwd",
    "embedding",
    "embedding_bwd_",
    "lmhead_logprob_entropy",
    "lmhead_backward",
    "attention_varlen",
    "attention_varlen_bwd",
    "paged_decode_attention",
    "kv_append_",
    "sample_tokens",
    "grpo_advantage",
    "gae_advantage",
]


def _ops():
    return native.ops()


# ----------------------------------------------------------------------------------------------- GEMM
_FETCH_RIDER = None


def set_fetch_rider(rider) -> None:
    """``rider.take(flops)`` is asked by every large GEMM whether it should carry a piece of a pending gather of sharded
    bytes (``ops.gemm_fetch``: an extra warp per CTA copies them from their owners' memory while the tensor pipe works);
    it answers ``(src_ptrs, dst, total_bytes, slice_bytes, chunk_begin, chunk_end)`` or None. ``None`` removes the rider."""
    global _FETCH_RIDER
    _FETCH_RIDER = rider


def gemm(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
         a_mn: bool = False, b_mn: bool = False, out_f32: bool = False, accumulate: bool = False,
         max_ctas: int = 0) -> torch.Tensor:
    """``D = A @ B^T (+bias)``; ``a_mn``/``b_mn`` mean the operand is stored transposed ([K, M] / [K, N])."""
    if a.is_cuda:
        if _FETCH_RIDER is not None and max_ctas == 0:
            M = a.shape[1] if a_mn else a.shape[0]
            K = a.shape[0] if a_mn else a.shape[1]
            N = b.shape[1] if b_mn else b.shape[0]
            if (M // 128) * (N // 256) >= 128:  # fills the machine without a K split: its CTAs can carry copy work
                job = _FETCH_RIDER.take(2.0 * M * N * K)
                if job is not None:
                    return _ops().gemm_fetch(a, b, bias, out, a_mn, b_mn, out_f32, accumulate, *job, -1, None, 2.0)
        return _ops().gemm(a, b, bias, out, a_mn, b_mn, out_f32, accumulate, max_ctas)
    A = a.t() if a_mn else a
    Bt = b if b_mn else b.t()
    d = A.float() @ Bt.float()
    if bias is not None:
        d = d + bias.float()
    if out is not None:
        if accumulate:
            out.add_(d.to(out.dtype))
        else:
            out.copy_(d.to(out.dtype))
        return out
    return d if out_f32 else d.to(a.dtype)


def gemm_row_ranges(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], ranges, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a @ w[w0 : w0 + rows]^T (+ bias[w0 : w0 + rows])`` for every ``(w0, rows)`` of ``ranges``, results side by side: the
    q | k | v (or gate | up) rows of one tensor-parallel rank inside the replicated fused weight. Up to 1024 tokens on the
    GPU run as one launch of the kernel for few tokens; otherwise one GEMM per range."""
    n = sum(int(r) for _, r in ranges)
    if out is None:
        out = torch.empty(a.shape[0], n, dtype=a.dtype, device=a.device)
    if a.is_cuda and a.shape[0] <= 1024 and len(ranges) <= 4:
        if _ops().gemm_row_ranges_(a, w, bias, [int(v) for pr in ranges for v in pr], out):
            return out
    col = 0
    for w0, rows in ranges:
        gemm(a, w[w0 : w0 + rows], bias[w0 : w0 + rows] if bias is not None else None, out=out[:, col : col + rows])
        col += rows
    return out


def _accumulate_wgrad(param: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor) -> Optional[torch.Tensor]:
    """dW += dy^T x into ``param.main_grad`` when present (returns None) else returns the gradient."""
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        gemm(dy2, x2, out=mg, a_mn=True, b_mn=True, out_f32=True, accumulate=True)
        return None
    return gemm(dy2, x2, a_mn=True, b_mn=True, out_f32=True).to(param.dtype)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.bias_ref = bias
        ctx.in_shape = x.shape
        y = gemm(x2, weight, bias)
        return y.reshape(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = gemm(dy2, weight, b_mn=True).reshape(ctx.in_shape) if ctx.needs_input_grad[0] else None
        dw = _accumulate_wgrad(weight, dy2, x2) if ctx.needs_input_grad[1] else None
        db = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            s = dy2.float().sum(0)
            mg = getattr(ctx.bias_ref, "main_grad", None)
            if mg is not None:
                mg.add_(s)
            else:
                db = s.to(dy.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    if x.is_cuda:
        return _Linear.apply(x, weight, bias)
    return F.linear(x, weight, bias)


# ----------------------------------------------------------------------------------------------- RMSNorm
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None):
    """Returns ``(y, x_eff, rstd)`` with ``x_eff = x (+ residual)`` (no autograd; see models.native)."""
    if x.is_cuda:
        return _ops().rmsnorm_fwd(x, residual, weight, eps)
    xe = x if residual is None else (x + residual)
    xf = xe.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
    y = (xf * rstd.unsqueeze(-1) * weight.float()).to(x.dtype)
    return y, xe, rstd.reshape(-1)


def rms_norm_bwd(dy, x, weight, rstd, dres_in, dw_out: torch.Tensor, accumulate: bool = True) -> torch.Tensor:
    if x.is_cuda:
        return _ops().rmsnorm_bwd(dy, x, weight, rstd, dres_in, dw_out, accumulate)
    H = x.shape[-1]
    xf, dyf, wf = x.float().reshape(-1, H), dy.float().reshape(-1, H), weight.float()
    rs = rstd.reshape(-1, 1)
    dot = (dyf * wf * xf).sum(-1, keepdim=True)
    dx = rs * dyf * wf - xf * (dot * rs.pow(3) / H)
    if dres_in is not None:
        dx = dx + dres_in.float().reshape(-1, H)
    dw = (dyf * xf * rs).sum(0)
    if accumulate:
        dw_out.add_(dw)
    else:
        dw_out.copy_(dw)
    return dx.to(x.dtype).reshape(x.shape)


# ----------------------------------------------------------------------------------------------- RoPE
def rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict] = None, max_position_embeddings: int = 0):
    """(inverse frequencies [head_dim/2] in fp64, factor on cos/sin) for plain rotary embeddings and their context
    extensions: ``linear`` (positions divided by ``factor``), ``llama3`` (long wavelengths divided by ``factor``, a smooth
    blend in the band between ``original / low_freq_factor`` and ``original / high_freq_factor``), ``yarn`` (interpolated
    low frequencies, extrapolated high ones, blended by a ramp between the dimensions that complete ``beta_fast`` and
    ``beta_slow`` turns inside the original context; cos/sin scaled by ``0.1 ln(factor) + 1`` unless given)."""
    dims = torch.arange(0, head_dim, 2, dtype=torch.float64)
    inv = 1.0 / (theta ** (dims / head_dim))
    kind = (scaling or {}).get("rope_type") or (scaling or {}).get("type") or "default"
    if kind == "default":
        return inv, 1.0
    factor = float(scaling.get("factor", 1.0))
    if kind == "linear":
        return inv / factor, 1.0
    original = int(scaling.get("original_max_position_embeddings") or max_position_embeddings)
    if kind == "llama3":
        lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        wavelen = 2 * math.pi / inv
        blend = ((original / wavelen - lo) / (hi - lo)).clamp(0.0, 1.0)   # 0: long wavelengths (scaled), 1: short ones (kept)
        return (1 - blend) * inv / factor + blend * inv, 1.0
    if kind == "yarn":
        fast, slow = float(scaling.get("beta_fast") or 32.0), float(scaling.get("beta_slow") or 1.0)

        def turns_dim(turns: float) -> float:   # dimension whose wavelength makes ``turns`` rotations over the original context
            return head_dim * math.log(original / (turns * 2 * math.pi)) / (2 * math.log(theta))

        low, high = turns_dim(fast), turns_dim(slow)
        if scaling.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, head_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(head_dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0.0, 1.0)
        inv = inv / factor * ramp + inv * (1 - ramp)
        att = scaling.get("attention_factor")
        if att is None:
            def mscale(f, m=1.0):
                return 1.0 if f <= 1 else 0.1 * m * math.log(f) + 1.0

            ms, ms_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
            att = mscale(factor, ms) / mscale(factor, ms_all) if ms and ms_all else mscale(factor)
        return inv, float(att)
    raise NotImplementedError(f"rope scaling type {kind!r}")


def rope_table(max_pos: int, head_dim: int, theta: float, device, scaling: Optional[dict] = None,
               max_position_embeddings: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables [max_pos, head_dim/2] in fp32 (HF rotate-half convention), context-extension rules folded in."""
    inv, att = rope_inv_freq(head_dim, theta, scaling, max_position_embeddings)
    ang = torch.arange(max_pos, dtype=torch.float64).unsqueeze(1) * inv.unsqueeze(0)
    return (ang.cos() * att).float().to(device), (ang.sin() * att).float().to(device)


def apply_rope_(x: torch.Tensor, positions: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor,
                backward: bool = False) -> torch.Tensor:
    """In-place rotation of ``x`` [T, heads, hd] (a strided view is fine)."""
    audit.check_index("apply_rope_", "positions", positions, cos_t.shape[0])
    if x.is_cuda:
        _ops().rope_(x, positions.to(torch.int32), cos_t, sin_t, backward)
        return x
    half = x.shape[-1] // 2
    c = cos_t[positions.long()].unsqueeze(1).to(torch.float32)
    s = sin_t[positions.long()].unsqueeze(1).to(torch.float32)
    if backward:
        s = -s
    a, b = x[..., :half].float().clone(), x[..., half:].float().clone()
    x[..., :half] = (a * c - b * s).to(x.dtype)
    x[..., half:] = (b * c + a * s).to(x.dtype)
    return x


# ----------------------------------------------------------------------------------------------- SwiGLU
def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    if gate_up.is_cuda:
        return _ops().swiglu_fwd(gate_up)
    g, u = gate_up.chunk(2, dim=-1)
    return F.silu(g) * u


FUSED_SWIGLU = os.environ.get("VERL_B200_FUSED_SWIGLU", "1") != "0"


def gemm_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, want_gate_up: bool = False):
    """``silu(x W_gate^T) * (x W_up^T)`` for the stacked weight ``[W_gate; W_up]``; returns ``(act, gate_up or None)``.
    Training-sized inputs on the GPU run the GEMM whose epilogue applies the activation (the [tokens, 2I] pre-activation
    is only written when ``want_gate_up``, for a backward pass that keeps it); decode-sized ones keep the kernel for few
    tokens plus the activation kernel."""
    if (x.is_cuda and FUSED_SWIGLU and x.dim() == 2 and x.shape[0] > 1024 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and w_gate_up.is_contiguous() and w_gate_up.shape[0] % 8 == 0 and w_gate_up.shape[1] % 8 == 0):
        act, gu = _ops().gemm_swiglu(x, w_gate_up, bool(want_gate_up))
        return act, (gu if want_gate_up else None)
    gu = gemm(x, w_gate_up)
    return swiglu(gu), (gu if want_gate_up else None)


def swiglu_bwd(dout: torch.Tensor, gate_up: torch.Tensor) -> torch.Tensor:
    if gate_up.is_cuda:
        return _ops().swiglu_bwd(dout, gate_up)
    g, u = gate_up.float().chunk(2, dim=-1)
    d = dout.float()
    sg = torch.sigmoid(g)
    return torch.cat([d * u * sg * (1 + g * (1 - sg)), d * g * sg], dim=-1).to(gate_up.dtype)


# ----------------------------------------------------------------------------------------------- embedding
def embedding(ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    audit.check_index("embedding", "ids", ids, weight.shape[0])
    if weight.is_cuda:
        return _ops().embedding_fwd(ids.reshape(-1).contiguous(), weight)
    return F.embedding(ids.reshape(-1), weight)


DETERMINISTIC_ATTENTION = False  # set by enable_full_determinism(): order-stable accumulation instead of atomics / fused library back-ends


def embedding_bwd_(ids: torch.Tensor, dout: torch.Tensor, dweight: torch.Tensor) -> None:
    audit.check_index("embedding_bwd_", "ids", ids, dweight.shape[0])
    if dout.is_cuda and DETERMINISTIC_ATTENTION:
        # deterministic mode: the kernel adds repeated token ids with atomics; the sorted accumulation is order-stable
        dweight.index_add_(0, ids.reshape(-1), dout.to(dweight.dtype))
    elif dout.is_cuda:
        _ops().embedding_bwd_(ids.reshape(-1).contiguous(), dout.contiguous(), dweight)
    else:
        dweight.index_add_(0, ids.reshape(-1), dout.to(dweight.dtype))


# ----------------------------------------------------------------------------------------------- LM head
def _torch_logprob_entropy(hidden, weight, labels, inv_temp: float, chunk: int = 2048):
    lps, ents, lses = [], [], []
    for s in range(0, hidden.shape[0], chunk):
        logits = (hidden[s : s + chunk].float() @ weight.float().t()) * inv_temp
        lse = torch.logsumexp(logits, -1)
        p = torch.softmax(logits, -1)
        lps.append(logits.gather(-1, labels[s : s + chunk].unsqueeze(-1)).squeeze(-1) - lse)
        ents.append(lse - (p * logits).sum(-1))
        lses.append(lse)
    return torch.cat(lps), torch.cat(ents), torch.cat(lses)


def lmhead_logprob_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                           temperature: float = 1.0):
    """(logprob, entropy, lse), each fp32 [T], of ``labels`` under ``softmax(hidden @ weight^T / T)``."""
    inv_temp = 1.0 / max(float(temperature), 1e-8)
    audit.check_index("lmhead_logprob_entropy", "labels", labels, weight.shape[0])
    if hidden.is_cuda:
        return _ops().lmhead_fwd(hidden, weight, labels.contiguous(), inv_temp)
    return _torch_logprob_entropy(hidden, weight, labels, inv_temp)


def lmhead_logprob_entropy_vocab_parallel(hidden: torch.Tensor, weight_shard: torch.Tensor, labels: torch.Tensor,
                                          temperature: float, vocab_start: int, group):
    """Vocabulary-parallel fused head: every rank of ``group`` holds rows ``[vocab_start, vocab_start + V_local)`` of the
    head and runs the fused log-prob / entropy kernel on its slice; the slices are combined from three [T] vectors per rank
    (local LSE, label logit, expected logit), so no logits ever cross the link. Returns the global (logprob, entropy, lse).

    Parity target: ``verl/utils/megatron/tensor_parallel.py`` (``vocab_parallel_log_probs_from_logits``,
    ``vocab_parallel_entropy``)."""
    import torch.distributed as dist

    Vl = weight_shard.shape[0]
    local = labels - vocab_start
    mine = (local >= 0) & (local < Vl)
    lp_l, ent_l, lse_l = lmhead_logprob_entropy(hidden, weight_shard, torch.where(mine, local, torch.zeros_like(local)), temperature)
    n = dist.get_world_size(group)
    all_lse = torch.empty(n, lse_l.numel(), dtype=lse_l.dtype, device=lse_l.device)
    if lse_l.is_cuda:
        dist.all_gather_into_tensor(all_lse, lse_l.contiguous(), group=group)
    else:
        dist.all_gather(list(all_lse.unbind(0)), lse_l.contiguous(), group=group)
    lse = torch.logsumexp(all_lse, dim=0)
    share = torch.exp(lse_l - lse)                              # probability mass of this rank's slice
    pack = torch.stack([torch.where(mine, lp_l + lse_l, torch.zeros_like(lp_l)), share * (lse_l - ent_l)])
    dist.all_reduce(pack, group=group)
    return pack[0] - lse, lse - pack[1], lse


def lmhead_backward(hidden, weight, labels, temperature, lse, entropy, g_lp, g_ent, dweight_out: Optional[torch.Tensor],
                    vocab_chunk: int = 9728, vocab_start: int = 0):
    """Returns d_hidden (same dtype as hidden) and accumulates d_weight into ``dweight_out`` (fp32 [V, H]); a frozen head
    (``dweight_out`` None) skips the weight-gradient GEMMs. With a vocabulary-parallel head, ``weight`` is this rank's
    slice starting at ``vocab_start`` while ``lse`` / ``entropy`` are the global values: the result is this rank's partial
    d_hidden (to be summed over the group)."""
    inv_temp = 1.0 / max(float(temperature), 1e-8)
    T, H = hidden.shape
    V = weight.shape[0]
    if not hidden.is_cuda:
        logits = (hidden.float() @ weight.float().t()) * inv_temp
        p = torch.exp(logits - lse.unsqueeze(1))
        local = labels - vocab_start
        mine = ((local >= 0) & (local < V)).unsqueeze(1)
        onehot = torch.zeros_like(p).scatter_(1, local.clamp(0, V - 1).unsqueeze(1), 1.0) * mine
        dl = g_lp.unsqueeze(1) * (onehot - p)
        if g_ent is not None:
            ex = (lse - entropy).unsqueeze(1)
            dl = dl - g_ent.unsqueeze(1) * p * (logits - ex)
        dl = dl * inv_temp
        if dweight_out is not None:
            dweight_out.add_(dl.t() @ hidden.float())
        return (dl @ weight.float()).to(hidden.dtype)
    ops = _ops()
    ex = (lse - entropy).contiguous() if g_ent is not None else None
    g_lp = g_lp.float().contiguous()
    g_ent = g_ent.float().contiguous() if g_ent is not None else None
    dh = torch.zeros(T, H, device=hidden.device, dtype=torch.float32)
    buf = torch.empty(T, min(vocab_chunk, V), device=hidden.device, dtype=hidden.dtype)
    for v0 in range(0, V, vocab_chunk):
        v1 = min(V, v0 + vocab_chunk)
        wc = weight[v0:v1]
        dl = buf[:, : v1 - v0]
        ops.lmhead_dlogits(hidden, wc, labels, vocab_start + v0, inv_temp, lse, ex, g_lp, g_ent, dl)
        # d_hidden += dl @ W[v0:v1]      (B stored [K=Vc, N=H] -> MN-major)
        gemm(dl, wc, out=dh, b_mn=True, out_f32=True, accumulate=True)
        # d_W[v0:v1] += dl^T @ hidden
        if dweight_out is not None:
            gemm(dl, hidden, out=dweight_out[v0:v1], a_mn=True, b_mn=True, out_f32=True, accumulate=True)
    return dh.to(hidden.dtype)


# ----------------------------------------------------------------------------------------------- attention
def _sdpa_varlen(q, k, v, cu_seqlens, scale):
    """Causal attention over packed sequences through torch SDPA (per equal-length group)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    lens = (cu_seqlens[1:] - cu_seqlens[:-1]).tolist()
    out = torch.empty_like(q)
    uniform = len(set(lens)) == 1
    if uniform and len(lens) > 0:
        B, S = len(lens), lens[0]
        qq = q.reshape(B, S, nh, hd).transpose(1, 2)
        kk = k.reshape(B, S, nkv, hd).transpose(1, 2)
        vv = v.reshape(B, S, nkv, hd).transpose(1, 2)
        o = F.scaled_dot_product_attention(qq, kk, vv, is_causal=True, scale=scale, enable_gqa=nkv != nh)
        return o.transpose(1, 2).reshape(T, nh, hd)
    s0 = 0
    for n in lens:
        qq = q[s0 : s0 + n].transpose(0, 1).unsqueeze(0)
        kk = k[s0 : s0 + n].transpose(0, 1).unsqueeze(0)
        vv = v[s0 : s0 + n].transpose(0, 1).unsqueeze(0)
        o = F.scaled_dot_product_attention(qq, kk, vv, is_causal=True, scale=scale, enable_gqa=nkv != nh)
        out[s0 : s0 + n] = o.squeeze(0).transpose(0, 1)
        s0 += n
    return out


_ATTN_IMPL = {"fwd": None, "bwd": None}


def register_attention_impl(fwd=None, bwd=None) -> None:
    """Install native varlen attention kernels (called by ops.attention when the library provides them)."""
    if fwd is not None:
        _ATTN_IMPL["fwd"] = fwd
    if bwd is not None:
        _ATTN_IMPL["bwd"] = bwd


def attention_varlen(q, k, v, cu_seqlens, max_seqlen: int, scale: Optional[float] = None):
    """Causal GQA attention over packed sequences. q [T, nh, hd], k/v [T, nkv, hd]. Returns (out, lse|None)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if q.is_cuda and _ATTN_IMPL["fwd"] is not None and q.shape[-1] in (64, 128) and q.dtype == torch.bfloat16:
        return _ATTN_IMPL["fwd"](q, k, v, cu_seqlens.to(q.device), max_seqlen, scale)
    return _sdpa_varlen(q, k, v, cu_seqlens, scale), None


def attention_varlen_bwd(dout, q, k, v, out, lse, cu_seqlens, max_seqlen: int, scale: Optional[float] = None):
    """Returns (dq, dk, dv)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if q.is_cuda and _ATTN_IMPL["bwd"] is not None and lse is not None and q.shape[-1] == 128 and q.dtype == torch.bfloat16:
        return _ATTN_IMPL["bwd"](dout, q, k, v, out, lse, cu_seqlens.to(q.device), max_seqlen, scale)
    import contextlib

    ctx = contextlib.nullcontext()
    if DETERMINISTIC_ATTENTION and q.is_cuda:
        from torch.nn.attention import SDPBackend, sdpa_kernel

        ctx = sdpa_kernel(SDPBackend.MATH)  # the fused library back-ends accumulate dQ / dK in a run-dependent order
    with torch.enable_grad(), ctx:
        q_, k_, v_ = (t.detach().requires_grad_(True) for t in (q, k, v))
        o = _sdpa_varlen(q_, k_, v_, cu_seqlens, scale)
        return torch.autograd.grad(o, (q_, k_, v_), dout)


def _attention_query_slice(q, k, v, cu_seqlens, q_start: int, scale: float):
    T_q = q.shape[0]
    nh, nkv = q.shape[1], k.shape[1]
    cu = cu_seqlens.tolist()
    parts = []
    lo, hi = q_start, q_start + T_q
    for s0, s1 in zip(cu[:-1], cu[1:]):
        a, b = max(lo, s0), min(hi, s1)
        if a >= b:
            continue
        qq = q[a - lo : b - lo].transpose(0, 1).unsqueeze(0)          # [1, nh, b - a, hd]
        kk = k[s0:b].transpose(0, 1).unsqueeze(0)                     # keys from the start of the sequence to the last query
        vv = v[s0:b].transpose(0, 1).unsqueeze(0)
        # query i (stream position a + i) sees keys s0 .. a + i: a causal mask aligned to the bottom-right corner
        mask = torch.ones(b - a, b - s0, dtype=torch.bool, device=q.device).tril(diagonal=a - s0)
        o = F.scaled_dot_product_attention(qq, kk, vv, attn_mask=mask, scale=scale, enable_gqa=nkv != nh)
        parts.append(o.squeeze(0).transpose(0, 1))
    covered = sum(p.shape[0] for p in parts)
    if covered < T_q:  # rows past the end of the packed stream (padding): no keys, zero output
        parts.append(q.new_zeros(T_q - covered, nh, q.shape[2]) + 0 * q[covered:])
    return torch.cat(parts, 0)


def attention_query_slice(q, k, v, cu_seqlens, q_start: int, scale: Optional[float] = None):
    """Causal GQA attention of a contiguous slice of the packed stream's queries (``q`` [Tq, nh, hd] = stream positions
    ``q_start .. q_start + Tq``) against the keys / values of the WHOLE stream (``k``/``v`` [T, nkv, hd]): what one rank
    of a context-parallel group computes after the keys and values have been gathered. Every query attends to the keys
    of its own sequence up to itself. Library attention per sequence (a functional path, not a tuned kernel)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    with torch.no_grad():
        return _attention_query_slice(q, k, v, cu_seqlens, int(q_start), scale)


def attention_query_slice_bwd(dout, q, k, v, cu_seqlens, q_start: int, scale: Optional[float] = None):
    """(dq [Tq, nh, hd], dk [T, nkv, hd], dv [T, nkv, hd]) of :func:`attention_query_slice`; dk / dv are this rank's
    contributions for the whole stream and still have to be summed over the group."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    with torch.enable_grad():
        q_, k_, v_ = (t.detach().requires_grad_(True) for t in (q, k, v))
        o = _attention_query_slice(q_, k_, v_, cu_seqlens, int(q_start), scale)
        return torch.autograd.grad(o, (q_, k_, v_), dout, allow_unused=True)


def attention_with_prefix(q, k, v, k_prefix, v_prefix, cu_seqlens, prefix_lens, scale: Optional[float] = None):
    """Causal GQA attention of packed sequences whose first ``prefix_lens[i]`` positions are already in a cache: ``q``/``k``/
    ``v`` [T, heads, hd] hold the new tokens only (``cu_seqlens`` over them), ``k_prefix``/``v_prefix`` [sum(prefix_lens), nkv, hd]
    the cached keys / values in sequence order. Every new token attends to its sequence's whole prefix and to the new tokens up
    to itself. Library attention per sequence (the path of a prefix-cache hit at prefill; forward only)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    nh, nkv = q.shape[1], k.shape[1]
    cu = cu_seqlens.tolist()
    out = torch.empty_like(q)
    p0 = 0
    with torch.no_grad():
        for i, (s0, s1) in enumerate(zip(cu[:-1], cu[1:])):
            m, n = int(prefix_lens[i]), s1 - s0
            kk = torch.cat([k_prefix[p0 : p0 + m], k[s0:s1]], 0).transpose(0, 1).unsqueeze(0)
            vv = torch.cat([v_prefix[p0 : p0 + m], v[s0:s1]], 0).transpose(0, 1).unsqueeze(0)
            qq = q[s0:s1].transpose(0, 1).unsqueeze(0)
            mask = torch.ones(n, m + n, dtype=torch.bool, device=q.device).tril(diagonal=m)
            o = F.scaled_dot_product_attention(qq, kk, vv, attn_mask=mask, scale=scale, enable_gqa=nkv != nh)
            out[s0:s1] = o.squeeze(0).transpose(0, 1)
            p0 += m
    return out


def kv_append_(k, v, slots, k_cache, v_cache) -> None:
    audit.check_index("kv_append_", "slots", slots, k_cache.numel() // (k_cache.shape[-2] * k_cache.shape[-1]), skip_negative=True)
    if k.is_cuda:
        _ops().kv_append_(k, v, slots, k_cache.view(-1, k_cache.shape[-2], k_cache.shape[-1]),
                          v_cache.view(-1, v_cache.shape[-2], v_cache.shape[-1]))
        return
    kc = k_cache.view(-1, k_cache.shape[-2], k_cache.shape[-1])
    vc = v_cache.view(-1, v_cache.shape[-2], v_cache.shape[-1])
    ok = slots >= 0
    kc[slots[ok]] = k[ok]
    vc[slots[ok]] = v[ok]


def rope_kv_append_(qkv: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, slots: torch.Tensor,
                    k_cache: torch.Tensor, v_cache: torch.Tensor, nh: int, nkv: int, hd: int) -> None:
    """Decode-step fusion: rotate the q and k heads of ``qkv`` [T, (nh + 2 nkv) * hd] in place and append the rotated k
    and v rows to the paged caches at ``slots`` (negative: skip the append). One kernel on a GPU; the same three steps
    through the separate ops elsewhere."""
    if audit.enabled():
        audit.check_index("rope_kv_append_", "pos", pos, cos.shape[0])
        audit.check_index("rope_kv_append_", "slots", slots, k_cache.numel() // (nkv * hd), skip_negative=True)
        audit.check_aligned("rope_kv_append_", "qkv", qkv)
    if qkv.is_cuda and qkv.dtype == torch.bfloat16:
        _ops().rope_kv_append_(qkv, pos, cos, sin, slots, k_cache, v_cache, int(nh), int(nkv), int(hd))
        return
    T = qkv.shape[0]
    q = qkv[:, : nh * hd].view(T, nh, hd)
    k = qkv[:, nh * hd : (nh + nkv) * hd].view(T, nkv, hd)
    v = qkv[:, (nh + nkv) * hd :].view(T, nkv, hd)
    apply_rope_(q, pos, cos, sin)
    apply_rope_(k, pos, cos, sin)
    kv_append_(k, v, slots, k_cache, v_cache)


def paged_decode_attention(q, k_cache, v_cache, block_table, ctx_len, scale: Optional[float] = None, groups=None):
    """One query token per sequence against a paged cache [num_blocks, block_size, nkv, hd].

    ``groups`` = (members int32 [NG, 8], grp_pages int32 [NG], skip int32 [B], workspace fp32, psplit, nsplit): sequences
    that share their leading pages (the samples of one prompt) have those pages read once per group by a kernel that
    holds every member's query heads, and only the rest of each context per sequence; same result as without."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    audit.check_paged_cache("paged_decode_attention", block_table, ctx_len, k_cache.shape[0], k_cache.shape[1])
    if q.is_cuda:
        if groups is not None:
            members, grp_pages, skip, ws, psplit, nsplit = groups
            return _ops().paged_decode_grouped(q, k_cache, v_cache, block_table, ctx_len, members, grp_pages, skip, scale,
                                               int(psplit), int(nsplit), ws)
        return _ops().paged_decode(q, k_cache, v_cache, block_table, ctx_len, scale)
    B, nh, hd = q.shape
    bs, nkv = k_cache.shape[1], k_cache.shape[2]
    out = torch.empty_like(q)
    for b in range(B):
        n = int(ctx_len[b])
        idx = torch.arange(n)
        rows = block_table[b, idx // bs].long() * bs + idx % bs
        kk = k_cache.view(-1, nkv, hd)[rows].float()
        vv = v_cache.view(-1, nkv, hd)[rows].float()
        g = nh // nkv
        kk = kk.repeat_interleave(g, dim=1)
        vv = vv.repeat_interleave(g, dim=1)
        s = torch.einsum("hd,thd->ht", q[b].float(), kk) * scale
        p = torch.softmax(s, -1)
        out[b] = torch.einsum("ht,thd->hd", p, vv).to(q.dtype)
    return out


# ----------------------------------------------------------------------------------------------- sampling
def sample_tokens(logits: torch.Tensor, temperature: float, seeds: torch.Tensor, step: int, valid_vocab: int = 0,
                  top_k: int = -1, top_p: float = 1.0):
    """Returns (tokens int64 [B], logprobs fp32 [B]) — the log-prob is of the processed distribution."""
    B, V = logits.shape
    vv = valid_vocab if 0 < valid_vocab <= V else V
    if logits.is_cuda and logits.dtype == torch.bfloat16:
        inv_temp = 0.0 if temperature <= 0 else 1.0 / temperature
        if (top_k <= 0 and top_p >= 1.0) or temperature <= 0:
            return _ops().sample(logits, vv, inv_temp, seeds, step)
        # filtered sampling stays on the device (and inside a captured decode graph): histogram selection, no sort
        return _ops().sample_topkp(logits, vv, inv_temp, int(top_k), float(top_p), seeds, step)
    x = logits[:, :vv].float()
    if temperature <= 0:
        tok = x.argmax(-1)
        return tok, torch.log_softmax(x, -1).gather(-1, tok.unsqueeze(-1)).squeeze(-1)
    x = x / temperature
    if top_k > 0:
        kth = torch.topk(x, min(top_k, vv), dim=-1).values[:, -1:]
        x = x.masked_fill(x < kth, float("-inf"))
    if top_p < 1.0:
        sx, si = torch.sort(x, dim=-1, descending=True)
        cp = torch.softmax(sx, -1).cumsum(-1)
        drop = cp - torch.softmax(sx, -1) > top_p
        sx = sx.masked_fill(drop, float("-inf"))
        x = torch.full_like(x, float("-inf")).scatter(1, si, sx)
    lp = torch.log_softmax(x, -1)
    # one random stream per row, keyed by that row's seed (as in the device kernel): what a request samples does not depend
    # on which other requests share its batch
    gen = torch.Generator(device="cpu")
    toks = []
    for i, sd in enumerate(seeds.tolist()):
        gen.manual_seed((int(sd) * 1000003 + int(step)) % (2**63 - 1))
        u = torch.rand(lp.shape[1], generator=gen).clamp_(min=1e-20).to(lp.device)
        toks.append(torch.argmax(lp[i] - torch.log(-torch.log(u))))   # Gumbel-max
    tok = torch.stack(toks)
    return tok, lp.gather(-1, tok.unsqueeze(-1)).squeeze(-1)


# ----------------------------------------------------------------------------------------------- advantages
def grpo_advantage(rewards: torch.Tensor, mask: torch.Tensor, group: torch.Tensor, num_groups: int,
                   eps: float = 1e-6, norm_by_std: bool = True):
    """Device GRPO outcome advantage. ``group`` is an int tensor of group ids in [0, num_groups)."""
    if rewards.is_cuda:
        return _ops().grpo_advantage(rewards.float().contiguous(), mask.float().contiguous(),
                                     group.to(torch.int32).contiguous(), num_groups, eps, norm_by_std)
    scores = rewards.float().sum(-1)
    adv = torch.zeros_like(scores)
    for g in range(num_groups):
        sel = group == g
        n = int(sel.sum())
        if n == 0:
            continue
        mean = scores[sel].mean() if n > 1 else scores.new_zeros(())
        std = scores[sel].std() if n > 1 else scores.new_ones(())
        adv[sel] = (scores[sel] - mean) / (std + eps) if norm_by_std else scores[sel] - mean
    return adv.unsqueeze(-1) * mask.float(), scores


def gae_advantage(rewards, values, mask, gamma: float, lam: float, whiten: bool = True):
    if rewards.is_cuda:
        return _ops().gae(rewards.float().contiguous(), values.float().contiguous(), mask.float().contiguous(),
                          gamma, lam, whiten)
    from ..trainer.ppo import core_algos

    return core_algos.compute_gae_advantage_return(rewards, values, mask, gamma, lam)


# ----------------------------------------------------------------------------------------------- native attention
def _native_attn_fwd(q, k, v, cu_seqlens, max_seqlen, scale):
    out, lse = _ops().attn_fwd(q, k, v, cu_seqlens.to(torch.int32), float(scale))
    return out, lse


def enable_native_attention(forward: bool = True, backward: bool = True) -> None:
    """Route varlen attention on CUDA through the tcgen05 kernels (forward; backward when available)."""
    if forward:
        _ATTN_IMPL["fwd"] = _native_attn_fwd
    if backward and hasattr(torch.ops.verl_b200, "attn_bwd"):
        _ATTN_IMPL["bwd"] = _native_attn_bwd


def _native_attn_bwd(dout, q, k, v, out, lse, cu_seqlens, max_seqlen, scale):
    return _ops().attn_bwd(dout.contiguous(), q, k, v, out, lse, cu_seqlens.to(torch.int32), int(max_seqlen), float(scale))


# On a GPU the tcgen05 kernels are the attention path: forward for head_dim 64 / 128, backward for head_dim 128 (other
# head sizes differentiate through the reference formulation). VERL_B200_NATIVE_ATTN_BWD=0 keeps the backward off.
import os as _os

if torch.cuda.is_available():
    _ATTN_IMPL["fwd"] = _native_attn_fwd
    if _os.environ.get("VERL_B200_NATIVE_ATTN_BWD", "1") != "0":
        _ATTN_IMPL["bwd"] = _native_attn_bwd


# ----------------------------------------------------------------------------------------------- fp8 block scaling
def fp8_quantize_1x128(x: torch.Tensor):
    """``x`` [R, C] (C % 128 == 0) -> (``q`` uint8 [R, C] holding e4m3 bits, ``scales`` fp32 [C/128, R]) with
    ``x ~= q * scale`` per 1x128 block, ``scale = amax / 448``. Parity target: ``verl/utils/kernel/fp8_kernel.py``
    (blockwise cast to fp8) with the 1x128 block shape for both operands."""
    if x.is_cuda:
        return _ops().fp8_quant_1x128(x.contiguous())
    R, C = x.shape
    xb = x.float().view(R, C // 128, 128)
    scale = xb.abs().amax(-1).clamp_min(1e-12) / 448.0
    q = (xb / scale.unsqueeze(-1)).to(torch.float8_e4m3fn).view(R, C)
    return q.view(torch.uint8), scale.t().contiguous()


def fp8_dequantize_1x128(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    R, C = q.shape
    return (q.view(torch.float8_e4m3fn).float().view(R, C // 128, 128) * scales.t().unsqueeze(-1)).view(R, C)


def fp8_quantize_128x128(w: torch.Tensor):
    """``w`` [R, C] -> (``q`` uint8 [R, C] holding e4m3 bits, ``scale_inv`` fp32 [ceil(R/128), ceil(C/128)]) with
    ``w ~= q * scale_inv`` per 128 x 128 block: the weight layout of block-scaled fp8 checkpoints (what an external
    inference engine loads). Parity target: ``verl/utils/kernel/fp8_kernel.py:53-108`` (blockwise cast)."""
    if w.is_cuda and w.dtype == torch.bfloat16:
        return _ops().fp8_quant_128x128(w.contiguous())
    R, C = w.shape
    Rb, Cb = (R + 127) // 128, (C + 127) // 128
    pad = torch.zeros(Rb * 128, Cb * 128, dtype=torch.float32, device=w.device)
    pad[:R, :C] = w.float()
    blocks = pad.view(Rb, 128, Cb, 128)
    scale = blocks.abs().amax(dim=(1, 3)).clamp(min=1e-12) / 448.0
    q = (blocks / scale[:, None, :, None]).to(torch.float8_e4m3fn).view(Rb * 128, Cb * 128)[:R, :C]
    return q.contiguous().view(torch.uint8), scale


def fp8_dequantize_128x128(q: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
    R, C = q.shape
    s = scale_inv.repeat_interleave(128, 0)[:R].repeat_interleave(128, 1)[:, :C]
    return q.view(torch.float8_e4m3fn).float() * s


def linear_fp8_grouped(x_rows: torch.Tensor, wq: torch.Tensor, w_scales: torch.Tensor, n_out: int, tile_expert: torch.Tensor,
                       num_mtiles: torch.Tensor) -> torch.Tensor:
    """Grouped expert linear in block-scaled fp8: ``x_rows`` [rows, K] (rows grouped by expert in 128-row aligned segments,
    padding rows zero), ``wq`` [E * n_out, K] e4m3 with scales [K/128, E * n_out]; the expert of every 128-row tile comes
    from ``tile_expert``. Activations are quantised per row and 128-wide K block on the fly."""
    if x_rows.is_cuda:
        xq, xs = _ops().fp8_quant_1x128(x_rows.contiguous())
        return _ops().gemm_fp8_blockscale_grouped(xq, xs, wq, w_scales, int(n_out), tile_expert, num_mtiles)
    xq, xs = fp8_quantize_1x128(x_rows)
    xd = fp8_dequantize_1x128(xq, xs)
    wd = fp8_dequantize_1x128(wq, w_scales).view(-1, n_out, x_rows.shape[1])
    out = torch.zeros(x_rows.shape[0], n_out, dtype=torch.float32)
    for t in range(int(num_mtiles.reshape(-1)[0])):
        out[t * 128 : (t + 1) * 128] = xd[t * 128 : (t + 1) * 128] @ wd[int(tile_expert[t])].t()
    return out.to(x_rows.dtype)


def linear_fp8(x: torch.Tensor, wq: torch.Tensor, w_scales: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ dequant(wq)^T`` with on-the-fly 1x128 quantisation of the activation and a block-scaled e4m3 tensor-core
    GEMM (fp32 accumulation per 128-wide K block)."""
    if x.is_cuda:
        xq, xs = _ops().fp8_quant_1x128(x.contiguous())
        return _ops().gemm_fp8_blockscale(xq, xs, wq, w_scales, bias)
    xq, xs = fp8_quantize_1x128(x)
    y = fp8_dequantize_1x128(xq, xs) @ fp8_dequantize_1x128(wq, w_scales).t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)
