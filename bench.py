#!/usr/bin/env python
"""Headline benchmark: GRPO step tokens/s on the Qwen2.5-7B architecture (random-init bf16, synthetic prompts).

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus 8 --steps K --warmup W

One GRPO step = rollout (prefill + decode of every response) + rule reward + old-policy and reference log-probs +
GRPO advantages + actor update (forward, backward, grad reduction, clipped AdamW) + weight hand-over to the
rollout engine.  Weak scaling: every GPU owns ``--prompts-per-gpu`` prompts x ``--n`` samples (64 x 5 by default,
i.e. 512 x 5 on 8 GPUs), prompts of 1024 uniform random tokens, responses of up to 2048 tokens.

One timed pass of K steps, bracketed by barrier + synchronize, CUDA events, max over ranks.  Every step's prompts
are staged host->device from pinned memory and its scores and metrics are read back: ``e2e`` is the span of the
whole loop, ``value`` the sum of per-step spans that start after the copy in and end before the read-back.  A
wall-clock budget (``--time-budget-s``) cuts the numbers of warm-up and timed steps to what fits; the result line
carries the numbers actually run, and a cumulative line is printed after every finished step.

``--impl reference`` reports why the reference cannot run in this environment (its import needs packages that are
not installed and cannot be installed offline).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=2)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="native", choices=["native", "reference"])
    p.add_argument("--model", default="qwen2.5-7b")
    p.add_argument("--prompts-per-gpu", type=int, default=64)
    p.add_argument("--samples-per-prompt", dest="n", type=int, default=5)
    p.add_argument("--prompt-len", type=int, default=1024)
    p.add_argument("--response-len", type=int, default=2048)
    p.add_argument("--max-token-len", type=int, default=16384, help="token budget of a training micro-batch")
    p.add_argument("--max-num-seqs", type=int, default=320)
    p.add_argument("--no-recompute", action="store_true")
    p.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                   help="cpu: development dry run of the control flow (gloo, fp32, host timers); not a measurement")
    p.add_argument("--time-budget-s", type=float, default=720.0,
                   help="wall-clock budget of the whole run in seconds, counted from process start (0 = none): after the first "
                        "warm-up step the numbers of warm-up and timed steps are cut to what still fits, keeping three warm-up "
                        "steps when that many were asked for; the result line reports the numbers actually run")
    p.add_argument("--rollout-tp", type=int, default=0,
                   help="rollout tensor-parallel size; 0 = the named configuration: 2 on two or more GPUs (1 on one GPU). "
                        "1 selects pure data-parallel rollout replicas")
    p.add_argument("--train-tp", type=int, default=1, help="tensor-parallel size of the training engine (strategy=megatron when tp*pp > 1)")
    p.add_argument("--train-pp", type=int, default=1, help="pipeline-parallel size of the training engine")
    p.add_argument("--train-ep", type=int, default=1, help="expert-parallel size of the training engine (mixture-of-experts models; "
                                                           "must equal the data-parallel size)")
    p.add_argument("--layers", type=int, default=0, help="development only: override the number of decoder layers (the result is "
                                                         "marked as a reduced model and is not a measurement of the named config)")
    p.add_argument("--no-prefix-sharing", action="store_true",
                   help="pack every sample's prompt separately in the log-prob / training passes and prefill it separately "
                        "(default: the n samples of a prompt share its tokens; results are identical)")
    p.add_argument("--offload", default="auto", choices=["auto", "on", "off"],
                   help="second Adam moment in pinned host memory (optimizer_offload), which leaves the GPU's memory to activations "
                        "instead of recomputation; auto = on one GPU, where the whole unsharded optimizer state would sit on it")
    p.add_argument("--critic", action="store_true", help="PPO with a critic of the same architecture and GAE instead of GRPO")
    return p.parse_args()


def reference_arm(args) -> None:
    """The unmodified reference lives in baseline/_ref (installed with --no-deps). Importing it needs ray, tensordict,
    hydra-core and omegaconf, none of which is installed or present in the offline wheelhouse."""
    sys.path.insert(0, os.path.join(REPO, "baseline", "_ref"))
    why = None
    try:
        import verl  # noqa: F401
        from verl.trainer import main_ppo  # noqa: F401
    except Exception as e:  # ModuleNotFoundError: ray / tensordict / hydra / omegaconf
        why = f"{type(e).__name__}: {e}"
    if why is None:
        why = "reference imports, but its PPO entry point needs a Ray cluster and vLLM server actors that are not provisioned here"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": f"reference cannot run offline on this image ({why})"}))


def _process_start_time() -> float:
    """Wall-clock time at which this process was created (imports count against the time budget)."""
    try:
        import psutil

        return psutil.Process().create_time()
    except Exception:
        return time.time()


class _HostEvent:
    """Host-clock stand-in for a CUDA event (``--device cpu`` dry runs)."""

    def __init__(self):
        self.t = 0.0

    def record(self):
        self.t = time.perf_counter()

    def synchronize(self):
        pass

    def elapsed_time(self, other) -> float:
        return (other.t - self.t) * 1e3


def build_config(args, world: int):
    if args.no_prefix_sharing:
        os.environ["VERL_B200_SHARE_PREFIX"] = "0"
    from verl_b200.trainer.config import CONFIG_DIR
    from verl_b200.utils.config import load_config

    gbs = args.prompts_per_gpu * world
    ov = [
        f"data.train_batch_size={gbs}", f"data.max_prompt_length={args.prompt_len}",
        f"data.max_response_length={args.response_len}", f"data.synthetic.num_prompts={gbs * 16}",
        f"data.synthetic.prompt_length={args.prompt_len}", "data.synthetic.vocab_low=3", "data.shuffle=false",
        f"actor_rollout_ref.model.path={args.model}", "actor_rollout_ref.model.load_weights=false",
        f"actor_rollout_ref.model.enable_gradient_checkpointing={'false' if args.no_recompute else 'true'}",
        f"actor_rollout_ref.rollout.n={args.n}", "actor_rollout_ref.rollout.temperature=1.0",
        f"actor_rollout_ref.rollout.max_num_seqs={min(args.max_num_seqs, args.prompts_per_gpu * args.n)}",
        "actor_rollout_ref.rollout.gpu_memory_utilization=0.45", "actor_rollout_ref.rollout.sync_interval=32",
        f"actor_rollout_ref.rollout.tensor_model_parallel_size={args.rollout_tp or (2 if world >= 2 and world % 2 == 0 else 1)}",
        f"actor_rollout_ref.actor.ppo_mini_batch_size={gbs}", "actor_rollout_ref.actor.use_dynamic_bsz=true",
        f"actor_rollout_ref.actor.ppo_max_token_len_per_gpu={args.max_token_len}",
        "actor_rollout_ref.actor.use_kl_loss=true", "actor_rollout_ref.actor.kl_loss_coef=0.001",
        "actor_rollout_ref.actor.optim.lr=1e-6", "algorithm.adv_estimator=grpo", "reward_model.reward_manager=token_rule",
        f"trainer.n_gpus_per_node={world}", "trainer.nnodes=1", "trainer.total_epochs=1000", "trainer.val_before_train=false",
        "trainer.resume_mode=disable", "trainer.save_freq=-1", "trainer.test_freq=-1", "trainer.logger=[]",
        "trainer.worker_group=spmd", f"trainer.device={args.device}",
    ]
    if args.offload == "on" or (args.offload == "auto" and world == 1 and args.train_tp * args.train_pp * args.train_ep == 1):
        # the second Adam moment alone (4 bytes per parameter) makes room for every layer's activations of a 7B model
        ov += ["actor_rollout_ref.actor.fsdp_config.optimizer_offload=true",
               "actor_rollout_ref.actor.fsdp_config.optimizer_offload_states=exp_avg_sq"]
    if args.layers > 0:
        ov += [f"+actor_rollout_ref.model.override_config.num_hidden_layers={args.layers}"]
    mp = args.train_tp * args.train_pp
    if mp * args.train_ep > 1:
        ov += ["actor@actor_rollout_ref.actor=megatron_actor",
               f"actor_rollout_ref.actor.megatron.tensor_model_parallel_size={args.train_tp}",
               f"actor_rollout_ref.actor.megatron.pipeline_model_parallel_size={args.train_pp}",
               f"actor_rollout_ref.actor.megatron.expert_model_parallel_size={args.train_ep}"]
    if args.critic:
        ov = [o for o in ov if not o.startswith(("algorithm.adv_estimator", "actor_rollout_ref.actor.use_kl_loss"))]
        ov += ["algorithm.adv_estimator=gae", "algorithm.gamma=1.0", "algorithm.lam=1.0", "actor_rollout_ref.actor.use_kl_loss=false",
               "actor_rollout_ref.actor.clip_ratio=0.2", f"critic.model.path={args.model}", "critic.model.load_weights=false",
               f"critic.ppo_mini_batch_size={gbs}", "critic.use_dynamic_bsz=true", f"critic.ppo_max_token_len_per_gpu={args.max_token_len}",
               "critic.optim.lr=1e-5"]
        if args.layers > 0:
            ov += [f"+critic.model.override_config.num_hidden_layers={args.layers}"]
        if mp > 1:
            ov += ["critic@critic=megatron_critic", f"critic.megatron.tensor_model_parallel_size={args.train_tp}",
                   f"critic.megatron.pipeline_model_parallel_size={args.train_pp}"]
    cfg = load_config(CONFIG_DIR, "ppo_trainer", ov)
    cfg.data.synthetic["vocab_high"] = None
    return cfg


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from verl_b200.models.config import get_preset
    from verl_b200.ops import native
    from verl_b200.trainer.ppo.ray_trainer import RayPPOTrainer
    from verl_b200.trainer.ppo.reward import load_reward_manager
    from verl_b200.single_controller.local import SPMDWorkerGroup
    from verl_b200.utils.distributed import initialize_global_process_group
    from verl_b200.utils.profiler.clocks import ClockSampler

    on_gpu = args.device == "cuda"
    if not on_gpu:
        os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    local_rank, rank, world = initialize_global_process_group()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run for N>1"
    dev = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")
    if on_gpu:
        native.load()
    Event = (lambda: torch.cuda.Event(enable_timing=True)) if on_gpu else _HostEvent
    launch_count = native.launch_count if on_gpu else (lambda: 0)
    check_status = native.check_status if on_gpu else (lambda: None)

    cfg = build_config(args, world)
    cfg.data.synthetic["vocab_high"] = get_preset(args.model).vocab_size
    reward_fn = load_reward_manager(cfg, None)
    trainer = RayPPOTrainer(config=cfg, tokenizer=None, ray_worker_group_cls=SPMDWorkerGroup, reward_fn=reward_fn,
                            val_reward_fn=None, device_name=args.device)
    trainer.init_workers()
    trainer.global_steps = 1
    it = iter(trainer.train_dataloader)

    def next_batch():
        nonlocal it
        try:
            return next(it)
        except StopIteration:
            it = iter(trainer.train_dataloader)
            return next(it)

    def sync():
        if world > 1:
            dist.barrier()
        if on_gpu:
            torch.cuda.synchronize()

    def to_pinned(batch):
        return {k: (v.pin_memory() if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}

    def to_device(batch):
        return {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}

    t_start = _process_start_time()

    def agree_max(x: float) -> float:
        """Same decision on every rank: the maximum over ranks of a host-side float."""
        if world == 1:
            return float(x)
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    # ---- warm-up: the first step is timed on the host to size the rest of the run against the wall-clock budget
    last_metrics = {}
    warmup, steps = max(args.warmup, 0), max(args.steps, 1)
    done_warm = 0
    step_s = 0.0
    if warmup > 0:
        sync()
        t0 = time.time()
        last_metrics, _ = trainer.train_step(next_batch())
        trainer.global_steps += 1
        sync()
        step_s = agree_max(time.time() - t0)
        done_warm = 1
    if args.time_budget_s > 0 and done_warm:
        left = args.time_budget_s - agree_max(time.time() - t_start) - 20.0  # 20 s for the report and teardown
        fit = max(1, int(left / (step_s * 1.03)))  # steps that still fit (the first one includes one-time captures)
        w_min = max(0, min(warmup, 3) - done_warm)
        steps = max(1, min(steps, fit - w_min))
        warmup = done_warm + max(0, min(warmup - done_warm, fit - steps))
    for _ in range(warmup - done_warm):
        last_metrics, _ = trainer.train_step(next_batch())
        trainer.global_steps += 1
    check_status()

    # ---- one timed pass.  Every step: prompts come from pinned host memory (H2D inside the end-to-end region), the
    # step runs through the trainer's public ``train_step``, the per-sample scores and the metric scalars are read
    # back (D2H inside the end-to-end region).  ``value`` sums per-step CUDA-event spans that start after the H2D copy
    # and end before the read-back; ``e2e`` is the span of the whole loop.
    sampler = ClockSampler(torch.cuda.current_device(), period_s=0.5) if rank == 0 and on_gpu else None
    if sampler:
        sampler.start()
    gbs = args.prompts_per_gpu * world
    ev = [(Event(), Event()) for _ in range(steps)]
    e_all0, e_all1 = Event(), Event()
    pin = (lambda t: t.pin_memory()) if on_gpu else (lambda t: t)
    # a tensor x pipeline parallel replica feeds the same rows to all of its ranks: a rank then holds (and reads back) the
    # replica's rows, and its tokens count once per replica
    dup = max(1, args.train_tp * args.train_pp)
    host_scores = pin(torch.empty(args.prompts_per_gpu * args.n * dup, dtype=torch.float32))
    tokens = h2d = d2h = 0
    reshard_s, phase_sum, grad_norms = 0.0, {}, []

    def report(k: int, partial: bool) -> None:
        """Collective over ranks; rank 0 prints one JSON line for the first ``k`` timed steps."""
        ms_dev = sum(ev[j][0].elapsed_time(ev[j][1]) for j in range(k))
        ms_all = e_all0.elapsed_time(e_all1)
        t = torch.tensor([ms_dev, ms_all], device=dev, dtype=torch.float64)
        tok = torch.tensor([float(tokens) / dup], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.all_reduce(tok)
        if rank != 0:
            return
        ms_dev, ms_all, tok_all = float(t[0]), float(t[1]), float(tok)
        rollout_tp = int(getattr(trainer.actor_rollout_wg.worker, "rollout_tp", 1))
        mp = args.train_tp * args.train_pp * args.train_ep
        out = {
            "metric": "GRPO step tokens/sec (prompt+response tokens of the step / step time, whole job)",
            "value": tok_all / (ms_dev / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": k, "warmup": warmup,
            "requested_steps": args.steps, "requested_warmup": args.warmup,
            "ms_per_step": ms_dev / k, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if on_gpu else "fp32 (cpu dry run)",
            "data": "synthetic (uniform random-token prompts, mod-7 rule reward, random-init weights)",
            "config": {"model": args.model, "global_batch": gbs * args.n, "prompts": gbs, "samples_per_prompt": args.n,
                       "seq_len": args.prompt_len + args.response_len, "prompt_len": args.prompt_len,
                       "response_len": args.response_len,
                       "parallelism": (f"dp{world} (sharded optimizer, replicated bf16 weights) + colocated rollout "
                                       f"tp{rollout_tp} x dp{world // rollout_tp} on in-place weight shards") if mp == 1
                       else (f"train tp{args.train_tp} x pp{args.train_pp} x dp{world // (args.train_tp * args.train_pp)}"
                             f"{' x ep' + str(args.train_ep) + ' (experts sharded over dp)' if args.train_ep > 1 else ''} + rollout tp{rollout_tp} "
                             f"on weights gathered from the shards each step"),
                       "algorithm": "ppo+critic+gae" if args.critic else "grpo",
                       **({"reduced_model_layers": args.layers} if args.layers > 0 else {}),
                       "shared_prompt_packing": not args.no_prefix_sharing,
                       "host_offload": ",".join(getattr(getattr(trainer.actor_rollout_wg.worker, "actor", None), "_offloaded_states", ())) or "none",
                       "kept_activation_layers": getattr(getattr(trainer.actor_rollout_wg.worker, "actor", None), "last_kept_layers", None),
                       "l2": "inputs_larger_than_L2 (15 GB of weights stream through every pass)",
                       "time_budget_s": args.time_budget_s,
                       "mean_response_len": last_metrics.get("response_length/mean")},
            "e2e": {"value": tok_all / (ms_all / 1e3), "unit": "tokens/s", "ms_per_step": ms_all / k,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "api": "RayPPOTrainer.train_step on prompts staged from pinned host memory; scores and metrics read back"},
            "reshard_ms_per_step": 1e3 * reshard_s / k,
            "grad_norm_per_step": [round(g, 4) for g in grad_norms[:k]],  # finite: the optimizer really stepped
            "gpu_launches": int(launch_count() - n0),
            "clocks": (sampler.stop() if not partial else sampler.snapshot()) if sampler else None,
            "phases_s": {name: round(v / k, 3) for name, v in phase_sum.items()},
        }
        opt_s = getattr(getattr(trainer.actor_rollout_wg.worker, "actor", None), "last_optimizer_step_s", None)
        if opt_s is not None:
            out["optimizer_step_s"] = round(float(opt_s), 3)  # the last step's, inside update_actor
        eng = getattr(trainer.actor_rollout_wg.worker, "rollout", None)
        st = getattr(eng, "stats", None)
        if isinstance(st, dict) and st.get("decode_steps"):
            # rank 0's rollout engine, cumulative since construction (warm-up steps included): where ``gen`` goes
            out["rollout_stats"] = {"decode_steps": int(st["decode_steps"]), "decode_gpu_ms_per_step": round(1e3 * st.get("decode_gpu_s", 0.0) / st["decode_steps"], 3),
                                    "prefill_tokens": int(st.get("prefill_tokens", 0)), "prefill_host_s": round(st.get("prefill_s", 0.0), 2),
                                    "kv_blocks": int(getattr(eng, "num_blocks", 0) or 0)}
        if partial:
            out["partial"] = True
        print(json.dumps(out), flush=True)

    sync()
    n0 = launch_count()
    e_all0.record()
    for i in range(steps):
        host = {k: (pin(v) if isinstance(v, torch.Tensor) else v) for k, v in next_batch().items()}
        batch = {k: (v.to(dev, non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in host.items()}
        h2d = sum(v.numel() * v.element_size() for v in host.values() if isinstance(v, torch.Tensor))
        ev[i][0].record()
        last_metrics, _ = trainer.train_step(batch)
        trainer.global_steps += 1
        ev[i][1].record()
        scores = trainer.last_batch.batch["token_level_scores"].sum(-1).float()
        host_scores[: scores.numel()].copy_(scores, non_blocking=True)
        if on_gpu:
            torch.cuda.current_stream().synchronize()
        d2h = scores.numel() * 4 + 8 * len([v for v in last_metrics.values() if isinstance(v, (int, float))])
        tokens += int(sum(trainer.last_batch.meta_info["global_token_num"]))
        reshard_s += float(last_metrics.get("timing_s/update_weights", 0.0))
        grad_norms.append(float(last_metrics.get("actor/grad_norm", float("nan"))))
        for k, v in last_metrics.items():
            if k.startswith("timing_s/") and isinstance(v, (int, float)):
                phase_sum[k.split("/", 1)[1]] = phase_sum.get(k.split("/", 1)[1], 0.0) + float(v)
        if i + 1 < steps:  # cumulative line after every finished step: a run cut short still leaves a result
            e_all1.record()
            e_all1.synchronize()
            report(i + 1, partial=True)
    e_all1.record()
    sync()
    report(steps, partial=False)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
