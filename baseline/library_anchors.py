#!/usr/bin/env python
"""Same-box timings of the libraries that the reference delegates its hot paths to.

The reference itself cannot run in this image (its import needs packages that are absent), so these numbers are
*library context*, not a reference measurement: they time

* ``vllm``       the rollout engine the reference launches (``verl/workers/rollout/vllm_rollout/vllm_async_server.py``):
                 offline engine, Qwen2.5-7B architecture with dummy weights, 64 random-token prompts of 1024 tokens x 5
                 samples, 2048 new tokens each, ``ignore_eos``, temperature 1.0: the generation phase of ``bench.py``;
* ``flash_attn`` the varlen attention the reference patches into its models (``verl/models/transformers/monkey_patch.py``):
                 forward + backward on the shape of ``verl_b200.ops.bench_kernels``' attention case;
* ``matmul``     ``torch.matmul`` (cuBLAS) on the GEMM shapes of the same table.

    python baseline/library_anchors.py --only vllm
    python baseline/library_anchors.py --only flash_attn,matmul

Every case prints one JSON line with its clock record.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)


def _clock_sampler(period_s: float):
    from verl_b200.utils.profiler.clocks import ClockSampler

    return ClockSampler(0, period_s=period_s).start()


def vllm_generation(args) -> None:
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    import torch

    from verl_b200.models.config import get_preset

    out = {"library": "vllm", "case": "generation phase of bench.py", "model": args.model, "prompts": args.prompts, "n": args.n,
           "prompt_len": args.prompt_len, "new_tokens": args.response_len}
    try:
        import vllm
        from vllm import LLM, SamplingParams

        out["version"] = vllm.__version__
        cfg_dir = tempfile.mkdtemp(prefix="anchor_cfg_")
        get_preset(args.model).save_pretrained(cfg_dir)
        llm = LLM(model=cfg_dir, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", seed=0,
                  max_model_len=args.prompt_len + args.response_len + 8, gpu_memory_utilization=0.85,
                  max_num_seqs=args.prompts * args.n, enforce_eager=False)
        g = torch.Generator().manual_seed(0)
        vocab = get_preset(args.model).vocab_size
        sp = SamplingParams(n=args.n, temperature=1.0, top_p=1.0, max_tokens=args.response_len, ignore_eos=True, detokenize=False)

        def batch():
            return [{"prompt_token_ids": torch.randint(3, vocab, (args.prompt_len,), generator=g).tolist()} for _ in range(args.prompts)]

        llm.generate(batch()[:8], SamplingParams(n=1, temperature=1.0, max_tokens=16, ignore_eos=True, detokenize=False), use_tqdm=False)
        times = []
        sampler = _clock_sampler(0.5)
        for _ in range(args.repeats):
            prompts = batch()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            res = llm.generate(prompts, sp, use_tqdm=False)
            torch.cuda.synchronize()
            times.append(time.perf_counter() - t0)
            new = sum(len(o.token_ids) for r in res for o in r.outputs)
        out.update(seconds=[round(t, 3) for t in times], new_tokens_generated=new,
                   new_tokens_per_s=round(new / min(times), 1),
                   step_tokens_per_s=round((new + args.prompts * args.n * args.prompt_len) / min(times), 1),
                   clocks=sampler.stop(), timing="host wall clock around LLM.generate, synchronised, best of repeats")
    except Exception as e:  # the library is optional context: report, do not fail
        out["error"] = f"{type(e).__name__}: {str(e)[:400]}"
    print(json.dumps(out), flush=True)


def flash_attn_varlen(args) -> None:
    import torch

    out = {"library": "flash_attn", "case": "causal varlen GQA attention forward + backward"}
    try:
        import flash_attn
        from flash_attn import flash_attn_varlen_func

        out["version"] = flash_attn.__version__
        dev = torch.device("cuda", 0)
        S, nseq, nh, nkv, hd = 3072, 5, 28, 4, 128
        T = S * nseq
        q, k, v = (torch.randn(T, h, hd, device=dev, dtype=torch.bfloat16, requires_grad=True) for h in (nh, nkv, nkv))
        do = torch.randn(T, nh, hd, device=dev, dtype=torch.bfloat16)
        cu = torch.arange(0, T + 1, S, dtype=torch.int32, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

        def fwd():
            return flash_attn_varlen_func(q, k, v, cu, cu, S, S, causal=True)

        def fwd_bwd():
            o = fwd()
            o.backward(do)

        rows = {}
        for name, fn in (("fwd", fwd), ("fwd_bwd", fwd_bwd)):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            sampler = _clock_sampler(0.01)
            tot = 0.0
            for _ in range(10):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                tot += e0.elapsed_time(e1)
            rows[name] = {"ms": round(tot / 10, 4), "clocks": sampler.stop()}
        out.update(shape=[nseq, S, nh, nkv, hd], **rows)
    except Exception as e:
        out["error"] = f"{type(e).__name__}: {str(e)[:400]}"
    print(json.dumps(out), flush=True)


def matmul_shapes(args) -> None:
    import torch

    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    H, I, tok = 3584, 18944, 16384
    for name, (M, N, K) in {"fwd_gate_up": (tok, 2 * I, H), "dgrad_down": (tok, I, H), "wgrad_qkv": (4608, H, tok), "decode_skinny": (320, 4608, H)}.items():
        a = (torch.randn(M, K, device=dev) * 0.05).bfloat16()
        b = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
        for _ in range(3):
            torch.matmul(a, b.t())
        torch.cuda.synchronize()
        sampler = _clock_sampler(0.01)
        tot = 0.0
        for _ in range(10):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b.t())
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        ms = tot / 10
        print(json.dumps({"library": "torch.matmul (cuBLAS)", "case": name, "shape": [M, N, K], "ms": round(ms, 4),
                          "tflops": round(2.0 * M * N * K / ms / 1e9, 1), "clocks": sampler.stop()}), flush=True)


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--only", default="vllm,flash_attn,matmul")
    p.add_argument("--model", default="qwen2.5-7b")
    p.add_argument("--prompts", type=int, default=64)
    p.add_argument("--n", type=int, default=5)
    p.add_argument("--prompt-len", type=int, default=1024)
    p.add_argument("--response-len", type=int, default=2048)
    p.add_argument("--repeats", type=int, default=2)
    a = p.parse_args()
    only = set(a.only.split(","))
    if "flash_attn" in only:
        flash_attn_varlen(a)
    if "matmul" in only:
        matmul_shapes(a)
    if "vllm" in only:
        vllm_generation(a)


if __name__ == "__main__":
    main()
