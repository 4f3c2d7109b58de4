"""Micro-benchmarks of the fused compute + collective kernels against their NCCL formulation (2 to 8 GPUs of one node).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m verl_b200.parallel.bench_fused

Every case is timed with CUDA events on the launching stream after warm-up, the time of an iteration is the MAX over
ranks, and rank 0 prints one JSON line per case with the roofline of the fused path: the slower of (FLOPs / measured
GEMM peak), (HBM bytes / measured copy bandwidth) and (bytes that must cross NVLink per GPU and direction / the measured
peer-copy bandwidth, 770 GB/s).
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0  # measured peer copy, one direction, per GPU


def _peaks() -> dict:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        d = json.load(open(os.path.join(here, "MEASURED_PEAKS.json")))
        out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    except Exception:
        pass
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--numel", type=int, default=1 << 28, help="elements of the gradient / parameter buffer (cases rs, ag)")
    a = ap.parse_args(argv)
    only = set(filter(None, a.only.split(",")))
    want = lambda name: not only or name in only

    from ..ops import native
    from ..ops import functional as F
    from ..utils.distributed import initialize_global_process_group
    from ..utils.profiler.clocks import ClockSampler
    from .symmetric import FusedRowParallelLinear, PeerBarrier, SymmetricBuffer

    initialize_global_process_group()
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    ops = native.ops()
    pk = _peaks()
    tag = "of measured" if pk["source"] == "measured" else "of fallback"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bar = PeerBarrier(dev)

    clock_log: list = []  # rank 0's SM clock record of every timed region since the last report

    def timed(fn) -> float:
        """Mean over iterations of the max over ranks of the device time of ``fn`` (ms)."""
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        per_iter = []
        sampler = ClockSampler(dev.index or 0, period_s=0.01).start() if rank == 0 else None
        for _ in range(a.iters):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            per_iter.append(e0.elapsed_time(e1))
        if sampler is not None:
            clock_log.append(sampler.stop())
        t = torch.tensor(per_iter, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.mean())

    def report(name, shape, ms_fused, ms_nccl, flops=0.0, hbm_bytes=0.0, link_bytes=0.0, **extra):
        floor_ms = max(flops / (pk["bf16_tflops"] * 1e9), hbm_bytes / (pk["hbm_gbs"] * 1e6), link_bytes / (NVLINK_GBS * 1e6))
        if rank == 0:
            print(json.dumps({"case": name, "world": world, "shape": shape, "ms_fused": round(ms_fused, 4),
                              "ms_nccl_formulation": None if ms_nccl is None else round(ms_nccl, 4),
                              "speedup": None if ms_nccl is None else round(ms_nccl / ms_fused, 3),
                              "roofline_ms": round(floor_ms, 4), "frac_of_roofline": round(floor_ms / ms_fused, 3),
                              "link_gbs": round(link_bytes / ms_fused / 1e6, 1),
                              "clocks": list(clock_log), **extra,
                              "denominators": f"{pk['bf16_tflops']} TFLOP/s, {pk['hbm_gbs']} GB/s {tag}; NVLink {NVLINK_GBS} GB/s per direction"}),
                  flush=True)
        clock_log.clear()

    n = (a.numel // (world * 1024)) * world * 1024
    shard = n // world
    lo = rank * shard

    if want("rs"):
        # gradient mean reduce-scatter + sum of squares of the reduced shard
        grads = SymmetricBuffer.allocate(n, torch.float32, dev)
        grads.tensor.normal_()
        out = torch.empty(shard, device=dev)
        ctrl = torch.zeros(4, device=dev)

        def fused():
            bar()
            ops.rs_sumsq_(grads.ptrs, 0, out, lo, rank, 1.0 / world, ctrl)
            bar()

        def nccl():
            dist.reduce_scatter_tensor(out, grads.tensor, op=dist.ReduceOp.AVG)
            ops.sumsq_(out, ctrl)

        t_nccl = timed(nccl)
        report("grad_reduce_scatter_sumsq", [n], timed(fused), t_nccl, hbm_bytes=4.0 * shard * (world + 1),
               link_bytes=4.0 * shard * (world - 1))
        if grads.multicast_ptr:
            # the same kernel through the NVSwitch multicast mapping: one multimem.ld_reduce returns the sum over the ranks,
            # so only the reduced shard crosses this GPU's link
            def fused_mc():
                bar()
                ops.rs_sumsq_(grads.ptrs, grads.multicast_ptr, out, lo, rank, 1.0 / world, ctrl)
                bar()

            report("grad_reduce_scatter_sumsq_multimem", [n], timed(fused_mc), t_nccl, hbm_bytes=4.0 * shard * 2,
                   link_bytes=4.0 * shard)
        del grads
    if want("ag"):
        # AdamW on the shard + publication of the new bf16 weights into every replica
        params = SymmetricBuffer.allocate(n, torch.bfloat16, dev)
        master, g = torch.randn(shard, device=dev), torch.randn(shard, device=dev)
        m, v = torch.zeros(shard, device=dev), torch.zeros(shard, device=dev)
        ctrl = torch.zeros(4, device=dev)
        ctrl[1] = 1.0
        flat = params.tensor

        def fused():
            bar()
            ops.adamw_allgather_(master, g, m, v, params.ptrs, 0, lo, rank, ctrl, 1e-5, 0.9, 0.999, 1e-8, 0.01, 1)
            bar()

        def nccl():
            ops.adamw_(master, g, m, v, flat[lo : lo + shard], ctrl, 1e-5, 0.9, 0.999, 1e-8, 0.01, 1, 1.0, False)
            dist.all_gather_into_tensor(flat, flat[lo : lo + shard].clone())

        t_nccl = timed(nccl)
        report("adamw_allgather_bf16", [n], timed(fused), t_nccl, hbm_bytes=shard * (4.0 * 7 + 2.0 * world),
               link_bytes=2.0 * shard * (world - 1))
        if params.multicast_ptr:
            def fused_mc():  # one multimem.st per 16 bytes reaches every replica: the shard leaves this GPU once
                bar()
                ops.adamw_allgather_(master, g, m, v, params.ptrs, params.multicast_ptr, lo, rank, ctrl, 1e-5, 0.9, 0.999, 1e-8, 0.01, 1)
                bar()

            report("adamw_allgather_bf16_multimem", [n], timed(fused_mc), t_nccl, hbm_bytes=shard * (4.0 * 7 + 2.0),
                   link_bytes=2.0 * shard)
        del params
    if want("gemm_ar"):
        # row-parallel linear (down projection of Qwen2.5-7B): partial GEMM + all-reduce
        N, K = 3584, 18944
        Kl = (K // world) // 64 * 64
        for M in (320, 8192):
            x = (torch.randn(M, Kl, device=dev) * 0.05).bfloat16()
            w = (torch.randn(N, Kl, device=dev) * 0.05).bfloat16()
            fl = FusedRowParallelLinear(max_rows=M, n=N, device=dev)
            y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

            def fused():
                fl(x, w, None, out=y)

            def nccl():
                F.gemm(x, w, out=y)
                dist.all_reduce(y)

            t_nccl = timed(nccl)
            report("row_parallel_gemm_allreduce", [M, N, Kl], timed(fused), t_nccl, flops=2.0 * M * N * Kl,
                   hbm_bytes=2.0 * (M * Kl + N * Kl + 2 * M * N), link_bytes=2.0 * M * N * (world - 1))
            if world > 2 and M > 1024:
                # the two in-kernel forms on their own (the default above picks per call size and group size), each checked
                # against the library formulation's result
                nccl()
                want_y = y.float().clone()
                for name, flag, link in (("one_kernel", False, 2.0 * M * N * (world - 1)),
                                         ("reduce_scatter_epilogue_then_allgather", True, 4.0 * M * N * (world - 1) / world)):
                    def form(flag=flag):
                        fl(x, w, None, out=y, two_shot=flag)

                    y.zero_()
                    form()
                    err = ((y.float() - want_y).norm() / want_y.norm()).item()
                    report(f"row_parallel_gemm_allreduce_{name}", [M, N, Kl], timed(form), t_nccl, flops=2.0 * M * N * Kl,
                           hbm_bytes=2.0 * (M * Kl + N * Kl + 2 * M * N), link_bytes=link, rel_err_vs_library=round(err, 5),
                           gemm_status=int(ops.gemm_status()))
            del fl
    if want("ag_gemm"):
        # fully sharded weight (equal slices on the ranks) gathered by the GEMM that consumes it, against all-gather + GEMM
        from .symmetric import PeerShardedLinear

        N, K, M = 37888, 3584, 8192   # gate_up projection of Qwen2.5-7B, 8192 tokens per rank
        lin = PeerShardedLinear(N, K, dev)
        lin.range.slice.view(torch.bfloat16).normal_(0, 0.05)
        lin.barrier()
        x = (torch.randn(M, K, device=dev) * 0.05).bfloat16()
        y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        per = lin.range.slice_bytes // 2
        w_pad = torch.empty(world * per, device=dev, dtype=torch.bfloat16)

        def fused():
            lin(x, None, out=y)

        def nccl():
            dist.all_gather_into_tensor(w_pad, lin.range.slice.view(torch.bfloat16))
            F.gemm(x, w_pad[: N * K].view(N, K), out=y)

        report("sharded_weight_gemm_fused_gather", [M, N, K], timed(fused), timed(nccl), flops=2.0 * M * N * K,
               hbm_bytes=2.0 * (M * K + N * K + M * N), link_bytes=2.0 * N * K * (world - 1) / world)
    if want("zero3_step"):
        # one optimizer round (2 micro-batches of 16k tokens, forward + backward + update) of a 6-layer slice of Qwen2.5-7B:
        # replicated working weights against weights sharded per unit, gathered by the GEMM kernels or by NCCL on a side stream
        from functools import partial

        from ..models.config import ModelConfig
        from ..workers.config import FSDPEngineConfig, OptimizerConfig
        from ..workers.engine.native.engine import NativeEngineWithLMHead
        from ..workers.utils.losses import sft_loss

        arch = ModelConfig(model_type="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=6,
                           num_attention_heads=28, num_key_value_heads=4, head_dim=128, eos_token_id=2, pad_token_id=0,
                           tie_word_embeddings=False, attention_bias=True)
        ids = torch.randint(3, 152064, (16, 2048), device=dev)
        am = torch.ones_like(ids)
        data = {"input_ids": ids, "attention_mask": am, "responses": ids[:, 512:], "response_mask": am[:, 512:]}
        rows = {}
        for name, stage, fz, fc in (("zero2_nccl_optimizer", 2, "1", "0"), ("zero3_gather_in_gemm", 3, "1", "0"), ("zero3_gather_nccl", 3, "0", "0")):
            os.environ["VERL_B200_ZERO3_FUSED"], os.environ["VERL_B200_FUSED_COMM"] = fz, fc
            eng = NativeEngineWithLMHead(arch, FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=8, zero_stage=stage,
                                                                enable_gradient_checkpointing=False),
                                         OptimizerConfig(lr=1e-6, clip_grad=1.0))
            eng.initialize()
            rows[name] = timed(lambda: eng.train_batch(dict(data), partial(sft_loss, None)))
            del eng
            torch.cuda.empty_cache()
        os.environ["VERL_B200_ZERO3_FUSED"] = os.environ["VERL_B200_FUSED_COMM"] = "1"
        if rank == 0:
            print(json.dumps({"case": "zero3_optimizer_round", "world": world, "tokens_per_rank": 2 * 16384, "layers": 6,
                              "ms": {k: round(v, 2) for k, v in rows.items()}, "clocks": list(clock_log)}), flush=True)
        clock_log.clear()
    if want("moe_ep"):
        # expert-parallel MoE layer of Qwen3-30B-A3B: router + dispatch + grouped GEMMs + combine
        from .expert_parallel import ExpertParallelMoE

        E, top_k, H, I, T = 128, 8, 2048, 768, 8192
        El = E // world
        h = (torch.randn(T, H, device=dev) * 0.5).bfloat16()
        gate = (torch.randn(E, H, device=dev) * 0.05).bfloat16()
        wgu = (torch.randn(El, 2 * I, H, device=dev) * 0.05).bfloat16()
        wd = (torch.randn(El, H, I, device=dev) * 0.05).bfloat16()
        ep = ExpertParallelMoE(E, top_k, H, max_tokens=T, device=dev)

        def fused():
            ep.forward(h, gate, wgu, wd)

        t_f = timed(fused)
        # every routed copy whose expert lives on another GPU crosses the link twice (dispatch and combine)
        link = 2.0 * T * top_k * H * (world - 1) / world
        report("moe_expert_parallel_layer_fwd", [T, H, E, top_k, I], t_f, None, flops=2.0 * T * top_k * 3 * H * I,
               hbm_bytes=2.0 * (El * 3 * H * I + 4 * T * top_k * H), link_bytes=link)
        if rank == 0 and int(ep.dropped) != 0:
            print(json.dumps({"case": "moe_expert_parallel_layer_fwd", "dropped_copies": int(ep.dropped)}))
    code_g, code_c = int(ops.gemm_status()), int(ops.comm_status())
    if code_g or code_c:
        raise RuntimeError(f"kernel status: gemm {code_g}, comm {code_c}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
