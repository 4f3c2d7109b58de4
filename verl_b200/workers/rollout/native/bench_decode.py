"""Decode-step micro-benchmark of the rollout engine: fills ``--seqs`` slots with contexts of ``--ctx`` tokens (KV
content is random; only the traffic matters) and times decode steps with CUDA events, eager or under the CUDA graph.

    python -m verl_b200.workers.rollout.native.bench_decode --model qwen2.5-7b --seqs 320 --ctx 2048 --steps 16

Prints one JSON line: ms per step, tokens/s, and the share of the HBM roofline (weights + KV bytes that a step must
read divided by the measured copy bandwidth).
"""

from __future__ import annotations

import argparse
import json

import torch

from ....models import FlatParams, get_preset
from .engine import RolloutEngine


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--seqs", type=int, default=320)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--eager", action="store_true", help="no CUDA graph (one launch per kernel, for launch lists)")
    ap.add_argument("--hbm-gbs", type=float, default=6545.6)
    ap.add_argument("--group", type=int, default=1, help="consecutive sequences that share the pages of their first --shared-ctx tokens")
    ap.add_argument("--shared-ctx", type=int, default=1024)
    ap.add_argument("--no-grouped-kernel", action="store_true",
                    help="with --group: keep the shared pages in the block tables but read them per sequence (plain decode kernel)")
    a = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    cfg = get_preset(a.model)
    P = FlatParams(cfg, dtype=torch.bfloat16, device=dev)
    P.init_weights(seed=1, std=0.02)
    bs = 64
    blocks_per_seq = (a.ctx + a.steps + a.warmup + 8 + bs - 1) // bs
    eng = RolloutEngine(cfg, P, max_num_seqs=a.seqs, max_model_len=blocks_per_seq * bs, block_size=bs,
                        num_blocks=a.seqs * blocks_per_seq, use_cuda_graph=not a.eager, eos_token_id=-1)
    eng.kv.normal_(0, 0.5)
    S = a.seqs
    eng.block_table[:, :blocks_per_seq] = torch.arange(S * blocks_per_seq, dtype=torch.int32, device=dev).view(S, blocks_per_seq)
    if a.group > 1:  # the samples of a prompt point at the same pages for the prompt part of their context
        shared_pages = min(a.shared_ctx, a.ctx) // bs
        lead = (torch.arange(S, device=dev) // a.group) * a.group
        eng.block_table[:, :shared_pages] = eng.block_table[lead, :shared_pages]
        if eng.grouped_decode and not a.no_grouped_kernel and a.group <= 8:
            # what the engine's admission does for the samples of a prompt: one decode group per prompt
            ng = S // a.group
            eng.grp_members[:ng, : a.group] = torch.arange(ng * a.group, dtype=torch.int32, device=dev).view(ng, a.group)
            eng.grp_pages[:ng] = shared_pages
            eng.seq_skip[: ng * a.group] = shared_pages
    eng.tok.fill_(5)
    eng.pos.fill_(a.ctx)
    eng.ctx.fill_(a.ctx + 1)
    eng.gen.fill_(1)
    eng.max_new.fill_(1 << 20)
    eng.active.fill_(True)
    eng.ignore_eos.fill_(True)
    eng._ensure_out(a.steps + a.warmup + 8)
    eng.temperature = 1.0
    eng._decode_steps(a.warmup)
    torch.cuda.synchronize()
    from ....utils.profiler.clocks import ClockSampler

    sampler = ClockSampler(dev.index or 0, period_s=0.02).start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    eng._decode_steps(a.steps)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / a.steps
    weight_bytes = (P.numel - (0 if cfg.tie_word_embeddings else cfg.vocab_size * cfg.hidden_size)) * 2
    kv_bytes = S * (a.ctx + a.steps // 2) * cfg.num_hidden_layers * 2 * cfg.kv_size * 2
    floor_ms = (weight_bytes + kv_bytes) / (a.hbm_gbs * 1e9) * 1e3
    print(json.dumps({"model": a.model, "seqs": S, "ctx": a.ctx, "graph": not a.eager, "ms_per_step": round(ms, 3),
                      "tokens_per_s": round(S / ms * 1e3, 1), "hbm_floor_ms": round(floor_ms, 3),
                      "fraction_of_hbm_roofline": round(floor_ms / ms, 3),
                      "group": a.group, "shared_ctx": a.shared_ctx if a.group > 1 else 0,
                      "grouped_kernel": bool(a.group > 1 and eng.grouped_decode and not a.no_grouped_kernel), "clocks": clocks}))


if __name__ == "__main__":
    main()
