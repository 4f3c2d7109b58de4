"""Micro-benchmarks of the native kernels with roofline fractions.

    python -m verl_b200.ops.bench_kernels                 # all kernels, default (training-sized) shapes
    python -m verl_b200.ops.bench_kernels --only gemm,attn_fwd --small   # a few hundred MB, for profiler captures

Every case is timed with CUDA events after warm-up, with an L2 flush (a 256 MB write) between iterations, and printed
as one JSON line: achieved TFLOP/s or GB/s and the fraction of the measured peak (``MEASURED_PEAKS.json`` at the
repository root when present, else the stated fallback).
"""

from __future__ import annotations

import argparse
import json
import math
import os

import torch

from ..utils.profiler.clocks import ClockSampler
from . import native


def _peaks() -> dict:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(here, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            out = {"hbm_gbs": float(d.get("hbm_gbs", out["hbm_gbs"])), "bf16_tflops": float(d.get("bf16_tflops", out["bf16_tflops"])),
                   "source": "measured"}
        except Exception:
            pass
    return out


class Timer:
    def __init__(self, dev, iters: int, warmup: int):
        self.dev, self.iters, self.warmup = dev, iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def __call__(self, fn) -> float:
        """Mean milliseconds per call; ``self.clocks`` holds the SM clock record of this timed region."""
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        sampler = ClockSampler(self.dev.index or 0, period_s=0.01).start()
        try:
            return self._timed(fn)
        finally:
            self.clocks = sampler.stop()

    def _timed(self, fn) -> float:
        total = 0.0
        for _ in range(self.iters):
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / self.iters


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--group", type=int, default=1, help="paged decode: sequences per group that share their prompt pages")
    a = ap.parse_args(argv)
    only = set(filter(None, a.only.split(",")))
    want = lambda name: not only or name in only
    dev = torch.device("cuda", 0)
    ops = native.ops()
    from . import functional as F

    pk = _peaks()
    T = Timer(dev, a.iters, a.warmup)
    tag = "of measured" if pk["source"] == "measured" else "of fallback"

    def report(name, shape, ms, flops=None, bytes_=None):
        rec = {"kernel": name, "shape": shape, "ms": round(ms, 4)}
        if flops is not None:
            tf = flops / ms / 1e9
            rec.update(tflops=round(tf, 1), frac=round(tf / pk["bf16_tflops"], 3), peak=f"{pk['bf16_tflops']} TFLOP/s {tag}")
        if bytes_ is not None:
            gbs = bytes_ / ms / 1e6
            rec.update(gbs=round(gbs, 1), frac_hbm=round(gbs / pk["hbm_gbs"], 3), hbm_peak=f"{pk['hbm_gbs']} GB/s {tag}")
        rec["clocks"] = getattr(T, "clocks", None)
        print(json.dumps(rec), flush=True)

    tok = 4096 if a.small else 16384
    H, I, V = 3584, 18944, 152064
    rnd = lambda *s: (torch.randn(*s, device=dev) * 0.05).bfloat16()

    if want("gemm") or want("gemm_decode"):
        for name, (M, N, K, amn, bmn) in {"gemm_fwd_gate_up": (tok, 2 * I if not a.small else 8192, H, False, False),
                                          "gemm_dgrad_down": (tok, I if not a.small else 8192, H, False, True),
                                          "gemm_wgrad_qkv": (4608, H, tok, True, True),
                                          "gemm_decode_skinny": (320, 4608, H, False, False)}.items():
            if not want("gemm") and name != "gemm_decode_skinny":
                continue
            A = rnd(K, M) if amn else rnd(M, K)
            B = rnd(K, N) if bmn else rnd(N, K)
            out = torch.empty(M, N, device=dev, dtype=torch.float32 if amn else torch.bfloat16)
            ms = T(lambda: ops.gemm(A, B, None, out, amn, bmn, amn, False, 0))
            report(name, [M, N, K], ms, flops=2.0 * M * N * K, bytes_=2.0 * (M * K + N * K) + out.element_size() * M * N)
    if want("gemm_decode_set"):
        # every GEMM of a decode step at 320 tokens (Qwen2.5-7B projections and LM head), with the library GEMM beside it
        for name, (M, N, K) in {"qkv": (320, 4608, H), "o": (320, H, H), "gate_up": (320, 2 * I, H), "down": (320, H, I),
                                "lm_head": (320, V, H), "qkv_64tok": (64, 4608, H), "down_tp2": (320, H, I // 2)}.items():
            A, B = rnd(M, K), rnd(N, K)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            ms = T(lambda: ops.gemm(A, B, None, out, False, False, False, False, 0))
            ck = T.clocks
            ms_lib = T(lambda: torch.matmul(A, B.t(), out=out))
            rec = {"kernel": f"gemm_decode_{name}", "shape": [M, N, K], "ms": round(ms, 4), "ms_library": round(ms_lib, 4),
                   "ratio_to_library": round(ms_lib / ms, 3), "weight_gbs": round(2.0 * N * K / ms / 1e6, 1),
                   "frac_hbm": round(2.0 * N * K / ms / 1e6 / pk["hbm_gbs"], 3), "splits": int(ops.gemm_skinny_splits(M, N, K)),
                   "clocks": {"ours": ck, "library": T.clocks}}
            print(json.dumps(rec), flush=True)
    if want("fp8"):
        # block-scaled e4m3 (1x128) linear against the bf16 GEMM on the same shapes: decode-sized and prefill-sized rows of
        # the Qwen2.5-7B projections. "fp8_total" includes the on-the-fly quantisation of the activation.
        for name, (M, N, K) in {"qkv_decode": (320, 4608, H), "gate_up_decode": (320, 2 * I, H), "down_decode": (320, H, I),
                                "gate_up_prefill": (tok, 2 * I if not a.small else 8192, H), "down_prefill": (tok, H, I if not a.small else 8192)}.items():
            x, w = rnd(M, K), rnd(N, K)
            wq, ws = F.fp8_quantize_1x128(w)
            xq, xs = F.fp8_quantize_1x128(x)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            ms_bf16 = T(lambda: ops.gemm(x, w, None, out, False, False, False, False, 0))
            c_bf16 = T.clocks
            ms_gemm = T(lambda: ops.gemm_fp8_blockscale(xq, xs, wq, ws, None))
            ms_total = T(lambda: F.linear_fp8(x, wq, ws))
            rec = {"kernel": f"fp8_blockscale_{name}", "shape": [M, N, K], "ms_bf16": round(ms_bf16, 4), "ms_fp8_gemm": round(ms_gemm, 4),
                   "ms_fp8_total": round(ms_total, 4), "speedup_gemm": round(ms_bf16 / ms_gemm, 3), "speedup_total": round(ms_bf16 / ms_total, 3),
                   "tflops_fp8_gemm": round(2.0 * M * N * K / ms_gemm / 1e9, 1),
                   "weight_gbs_fp8": round(N * K / ms_gemm / 1e6, 1), "weight_gbs_bf16": round(2.0 * N * K / ms_bf16 / 1e6, 1),
                   "clocks": {"bf16": c_bf16, "fp8": T.clocks}}
            print(json.dumps(rec), flush=True)
    if want("lmhead"):
        Vs = 32768 if a.small else V
        h, w = rnd(tok, H), rnd(Vs, H)
        labels = torch.randint(0, Vs, (tok,), device=dev)
        ms = T(lambda: ops.lmhead_fwd(h, w, labels, 1.0))
        report("lmhead_fwd_logprob_entropy", [tok, Vs, H], ms, flops=2.0 * tok * Vs * H)
    if want("attn_fwd") or want("attn_bwd"):
        S = 1024 if a.small else 3072
        nseq = max(1, tok // S)
        nh, nkv, hd = 28, 4, 128
        Tt = nseq * S
        q, k, v = rnd(Tt, nh, hd), rnd(Tt, nkv, hd), rnd(Tt, nkv, hd)
        cu = torch.arange(0, Tt + 1, S, dtype=torch.int32, device=dev)
        fl = 4.0 * nseq * nh * hd * S * S / 2
        if want("attn_fwd"):
            ms = T(lambda: ops.attn_fwd(q, k, v, cu, 1.0 / math.sqrt(hd)))
            report("attn_fwd_causal_gqa", [nseq, S, nh, nkv, hd], ms, flops=fl)
        if want("attn_bwd"):
            out, lse = ops.attn_fwd(q, k, v, cu, 1.0 / math.sqrt(hd))
            do = rnd(Tt, nh, hd)
            ms = T(lambda: ops.attn_bwd(do, q, k, v, out, lse, cu, S, 1.0 / math.sqrt(hd)))
            report("attn_bwd_causal_gqa", [nseq, S, nh, nkv, hd], ms, flops=2.5 * fl)

            def sdpa_bwd():
                with torch.enable_grad():
                    q_, k_, v_ = (t.detach().requires_grad_(True) for t in (q, k, v))
                    o = F._sdpa_varlen(q_, k_, v_, cu.cpu(), 1.0 / math.sqrt(hd))
                    torch.autograd.grad(o, (q_, k_, v_), do)

            ms = T(sdpa_bwd)
            report("library_sdpa_fwd_plus_bwd_for_comparison", [nseq, S, nh, nkv, hd], ms, flops=3.5 * fl)
    if want("paged_decode"):
        B_, ctx, bs = (64, 1024, 64) if a.small else (320, 2048, 64)
        nh, nkv, hd = 28, 4, 128
        nb = B_ * (ctx // bs)
        kc, vc = rnd(nb, bs, nkv, hd), rnd(nb, bs, nkv, hd)
        bt = torch.arange(nb, dtype=torch.int32, device=dev).view(B_, ctx // bs)
        cl = torch.full((B_,), ctx, dtype=torch.int32, device=dev)
        q = rnd(B_, nh, hd)
        ms = T(lambda: F.paged_decode_attention(q, kc, vc, bt, cl))
        report("paged_decode_attention", [B_, ctx, nh, nkv, hd], ms, bytes_=2.0 * 2 * nb * bs * nkv * hd)
        if a.group > 1:
            # the samples of a prompt share the pages of the first half of their context (one physical copy)
            shared = (ctx // 2) // bs
            lead = (torch.arange(B_, device=dev) // a.group) * a.group
            bt2 = bt.clone()
            bt2[:, :shared] = bt[lead, :shared]
            ms = T(lambda: F.paged_decode_attention(q, kc, vc, bt2, cl))
            uniq = 2.0 * 2 * bs * nkv * hd * ((B_ // a.group) * shared + B_ * (ctx // bs - shared))
            report(f"paged_decode_attention_shared_prefix_group{a.group}", [B_, ctx, nh, nkv, hd], ms, bytes_=uniq)
    if want("rmsnorm"):
        x, r, w = rnd(tok, H), rnd(tok, H), rnd(H)
        ms = T(lambda: F.rms_norm(x, w, 1e-6, r))
        report("rmsnorm_fwd_residual", [tok, H], ms, bytes_=2.0 * tok * H * 4)
        y, xe, rs = F.rms_norm(x, w, 1e-6, r)
        dw = torch.zeros(H, device=dev)
        ms = T(lambda: F.rms_norm_bwd(x, xe, w, rs, r, dw, True))
        report("rmsnorm_bwd", [tok, H], ms, bytes_=2.0 * tok * H * 4)
    if want("swiglu"):
        Is = 4096 if a.small else I
        gu = rnd(tok, 2 * Is)
        ms = T(lambda: F.swiglu(gu))
        report("swiglu_fwd", [tok, Is], ms, bytes_=2.0 * tok * Is * 3)
    if want("gemm_swiglu"):
        # up-projection of the gated MLP: GEMM with the activation in its epilogue against GEMM + activation kernel
        Is = 4096 if a.small else I
        x, w = rnd(tok, H), rnd(2 * Is, H)
        ms_f = T(lambda: ops.gemm_swiglu(x, w, False))
        ck = T.clocks
        ms_fk = T(lambda: ops.gemm_swiglu(x, w, True))
        ms_s = T(lambda: F.swiglu(ops.gemm(x, w, None, None, False, False, False, False, 0)))
        print(json.dumps({"kernel": "gemm_swiglu_fused", "shape": [tok, 2 * Is, H], "ms_fused": round(ms_f, 4),
                          "ms_fused_keep_preactivation": round(ms_fk, 4), "ms_gemm_plus_activation": round(ms_s, 4),
                          "tflops_fused": round(2.0 * tok * 2 * Is * H / ms_f / 1e9, 1), "speedup": round(ms_s / ms_f, 3),
                          "clocks": {"fused": ck, "separate": T.clocks}}), flush=True)
    if want("adamw"):
        n = (64 << 20) if a.small else (512 << 20)
        master, g = torch.randn(n, device=dev), torch.randn(n, device=dev)
        m, v2 = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        outb = torch.empty(n, device=dev, dtype=torch.bfloat16)
        ctrl = torch.zeros(4, device=dev)
        ctrl[1] = 1.0
        ms = T(lambda: ops.adamw_(master, g, m, v2, outb, ctrl, 1e-4, 0.9, 0.999, 1e-8, 0.01, 1, 1.0, False))
        report("adamw_fused_cast", [n], ms, bytes_=n * (4 * 4 + 3 * 4 + 2.0))
    if want("moe"):
        # one mixture-of-experts MLP of Qwen3-30B-A3B (128 experts, top-8, H 2048, I 768) on one GPU: router kernel,
        # expert-grouped layout, grouped tcgen05 GEMMs, weighted combine; backward adds grouped dgrad + wgrad
        from ..models import DecoderModel, FlatParams
        from ..models.config import ModelConfig

        Tm = 2048 if a.small else 8192
        cfg = ModelConfig(model_type="qwen3_moe", vocab_size=1024, hidden_size=2048, intermediate_size=6144, num_hidden_layers=1,
                          num_attention_heads=32, num_key_value_heads=4, head_dim=128, num_experts=128, num_experts_per_tok=8,
                          moe_intermediate_size=768, eos_token_id=2, pad_token_id=0, qk_norm=True, norm_topk_prob=True)
        P = FlatParams(cfg, dtype=torch.bfloat16, device=dev, with_main_grad=True)
        P.init_weights(seed=1, std=0.02)
        model = DecoderModel(cfg, P)
        W = P.layer(0)
        h2 = rnd(Tm, 2048) * 10
        g = rnd(Tm, 2048)
        fl = 2.0 * Tm * 8 * 3 * 2048 * 768
        ms = T(lambda: model._moe_fwd(W, h2, None))
        report("moe_layer_fwd_128e_top8", [Tm, 2048, 128, 8, 768], ms, flops=fl)

        def fwd_bwd():
            S = {}
            model._moe_fwd(W, h2, S)
            model._moe_bwd(W, g, h2, S)

        ms = T(fwd_bwd)
        report("moe_layer_fwd_bwd_128e_top8", [Tm, 2048, 128, 8, 768], ms, flops=3.0 * fl)
    native.check_status()


if __name__ == "__main__":
    main()
