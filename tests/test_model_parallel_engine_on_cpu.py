"""Tensor x pipeline parallel engine on gloo: loss, outputs, gradient norm and updated weights equal the unsharded engine."""
import os
import socket

import pytest
import torch


def _data(seed=0, b=4, L=24, R=16, V=500):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(3, V, (b, L), generator=g)
    am = torch.ones_like(ids)
    am[1, :3] = 0  # left padding on one row
    return {"input_ids": ids, "attention_mask": am, "responses": ids[:, -R:], "response_mask": am[:, -R:]}


def _arch(preset: str):
    """``name`` or ``name:L`` (the preset with L layers)."""
    import dataclasses

    from verl_b200.models import get_preset

    name, _, layers = preset.partition(":")
    cfg = get_preset(name)
    return dataclasses.replace(cfg, num_hidden_layers=int(layers)) if layers else cfg


def _proc(rank, world, port, tp, pp, q, ep=1, preset="tiny-llama", mbs=2, schedule="1f1b", sp=False, vpp=1):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                          VERL_ENGINE_DEVICE="cpu")
        from functools import partial

        from verl_b200.models import get_preset
        from verl_b200.utils.distributed import initialize_global_process_group
        from verl_b200.workers.config import McoreEngineConfig, OptimizerConfig
        from verl_b200.workers.engine.base import EngineRegistry
        from verl_b200.workers.utils.losses import sft_loss

        initialize_global_process_group()
        ec = McoreEngineConfig(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp, expert_model_parallel_size=ep, seed=7,
                               micro_batch_size_per_gpu=mbs if ep == 1 else (1 + rank // (tp * pp)))  # ep: unequal micro-batch counts get evened out
        object.__setattr__(ec, "pipeline_schedule", schedule)
        object.__setattr__(ec, "sequence_parallel", sp)
        if vpp > 1:
            object.__setattr__(ec, "virtual_pipeline_model_parallel_size", vpp)
        eng = EngineRegistry.new("language_model", "megatron", _arch(preset), ec, OptimizerConfig(lr=1e-2, clip_grad=0.05), device="cpu")
        eng.initialize()
        dp = eng.topo.dp
        data = _data()
        shard = {k: v.chunk(dp)[eng.topo.dp_rank] for k, v in data.items()}
        res = {"dp": dp, "tp_rank": eng.topo.tp_rank, "pp_rank": eng.topo.pp_rank}
        out = eng.train_batch(dict(shard), partial(sft_loss, None))
        res["grad_norm"] = float(out["metrics"]["grad_norm"])
        res["loss"] = float(out["loss"]) if "loss" in out else None
        inf = eng.infer_batch(dict(shard))
        res["log_probs"] = inf["model_output"]["log_probs"].float().numpy()  # by value: the child exits before the parent reads
        full = eng.gather_full_params()
        res["full"] = full.flat.float().numpy()
        q.put((rank, res))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def _run(world, tp, pp, ep=1, preset="tiny-llama", mbs=2, schedule="1f1b", sp=False, vpp=1):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_proc, args=(r, world, port, tp, pp, q, ep, preset, mbs, schedule, sp, vpp)) for r in range(world)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(world))
    for p in ps:
        p.join(timeout=30)
    for r in range(world):
        assert "error" not in res[r], res[r]["error"]
    return res


def _reference(preset="tiny-llama"):
    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from functools import partial

    from verl_b200.models import get_preset
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.utils.losses import sft_loss

    eng = NativeEngineWithLMHead(_arch(preset), FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=2), OptimizerConfig(lr=1e-2, clip_grad=0.05))
    eng.initialize()
    out = eng.train_batch(dict(_data()), partial(sft_loss, None))
    lp = eng.infer_batch(dict(_data()))["model_output"]["log_probs"]
    return float(out["metrics"]["grad_norm"]), lp, eng.params.flat.clone()


@pytest.mark.parametrize("world,tp,pp", [(2, 2, 1), (2, 1, 2), (4, 2, 2), (4, 1, 2)])
def test_model_parallel_engine_matches_unsharded(world, tp, pp):
    ref_norm, ref_lp, ref_flat = _reference()
    res = _run(world, tp, pp)
    dp = res[0]["dp"]
    for r in range(world):
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm), (r, res[r]["grad_norm"], ref_norm)
        got = torch.from_numpy(res[r]["full"])
        assert torch.allclose(got, ref_flat.float(), atol=3e-4), (r, (got - ref_flat.float()).abs().max())  # lr = 1e-2: a wrong gradient moves weights by ~1e-2
    rows = ref_lp.chunk(dp)
    for r in range(world):
        d = r // (tp * pp)
        assert torch.allclose(torch.from_numpy(res[r]["log_probs"]), rows[d], atol=1e-4), r


@pytest.mark.parametrize("world,tp,pp,vpp,layers,mbs", [(2, 1, 2, 2, 4, 1), (2, 1, 2, 3, 6, 2), (3, 1, 3, 2, 6, 1), (4, 2, 2, 2, 4, 1)])
def test_interleaved_pipeline_stages_match_unsharded(world, tp, pp, vpp, layers, mbs):
    """Virtual pipeline stages: every rank holds ``vpp`` chunks of the layer stack (chunk v of stage s = block v * pp + s)
    and a micro-batch goes ``vpp`` times round the ring; fewer (4 rows in 2) and more (4 rows in 4) micro-batches than
    stages; with tensor parallelism. Same update, log-probs and re-assembled full model as one process."""
    ref_norm, ref_lp, ref_flat = _reference(f"tiny-llama:{layers}")
    res = _run(world, tp, pp, preset=f"tiny-llama:{layers}", mbs=mbs, vpp=vpp)
    dp = res[0]["dp"]
    rows = ref_lp.chunk(dp)
    for r in range(world):
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm), (r, res[r]["grad_norm"], ref_norm)
        got = torch.from_numpy(res[r]["full"])
        assert torch.allclose(got, ref_flat.float(), atol=3e-4), (r, (got - ref_flat.float()).abs().max())
        assert torch.allclose(torch.from_numpy(res[r]["log_probs"]), rows[r // (tp * pp)], atol=1e-4), r


@pytest.mark.parametrize("world,pp,mbs,schedule", [(2, 2, 1, "1f1b"), (3, 3, 1, "1f1b"), (2, 2, 1, "gpipe")])
def test_pipeline_schedules_with_more_micro_batches_than_stages(world, pp, mbs, schedule):
    """Four micro-batches through two / three stages: warm-up, steady one-forward-one-backward and drain phases all run."""
    ref_norm, ref_lp, ref_flat = _reference()
    res = _run(world, 1, pp, mbs=mbs, schedule=schedule)
    for r in range(world):
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm), (r, res[r]["grad_norm"], ref_norm)
        got = torch.from_numpy(res[r]["full"])
        assert torch.allclose(got, ref_flat.float(), atol=3e-4), (r, (got - ref_flat.float()).abs().max())
        assert torch.allclose(torch.from_numpy(res[r]["log_probs"]), ref_lp, atol=1e-4), r


@pytest.mark.parametrize("world,tp,pp,preset", [(2, 2, 1, "tiny-llama"), (2, 2, 1, "tiny-qwen3"), (4, 2, 2, "tiny-llama")])
def test_sequence_parallel_inside_tensor_parallel_matches_unsharded(world, tp, pp, preset):
    """Token-sliced residual stream (all-gather / reduce-scatter around the projections); the packed batch has a token
    count that is not a multiple of the group size, so the padded tail is exercised too."""
    ref_norm, ref_lp, ref_flat = _reference(preset)
    res = _run(world, tp, pp, preset=preset, sp=True)
    dp = res[0]["dp"]
    rows = ref_lp.chunk(dp)
    for r in range(world):
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm), (r, res[r]["grad_norm"], ref_norm)
        got = torch.from_numpy(res[r]["full"])
        assert torch.allclose(got, ref_flat.float(), atol=3e-4), (r, (got - ref_flat.float()).abs().max())
        assert torch.allclose(torch.from_numpy(res[r]["log_probs"]), rows[r // (tp * pp)], atol=1e-4), r


def test_tensor_parallel_with_per_head_norms_matches_unsharded():
    """Qwen3-style q/k norms are applied per head: under tensor parallelism every rank sees a subset of the heads, so the
    gradients of these (replicated) weights are partial sums that must be completed over the group."""
    ref_norm, ref_lp, ref_flat = _reference("tiny-qwen3")
    res = _run(2, 2, 1, preset="tiny-qwen3")
    for r in range(2):
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm), (r, res[r]["grad_norm"], ref_norm)
        got = torch.from_numpy(res[r]["full"])
        assert torch.allclose(got, ref_flat.float(), atol=3e-4), (r, (got - ref_flat.float()).abs().max())


@pytest.mark.parametrize("world,tp,pp,preset", [(2, 2, 1, "tiny-moe"), (2, 2, 1, "tiny-qwen2-moe"), (4, 2, 2, "tiny-moe")])
def test_expert_tensor_parallel_matches_unsharded(world, tp, pp, preset):
    """Mixture-of-experts layers under tensor parallelism: every expert's (and the shared expert's) intermediate width is
    cut over the two ranks, the router stays whole. Same gradient norm, same updated full model (experts, router, shared
    expert gate re-assembled from the shards) and the same log-probs as one process."""
    ref_norm, ref_lp, ref_flat = _reference(preset)
    res = _run(world, tp, pp, preset=preset)
    dp = res[0]["dp"]
    rows = ref_lp.chunk(dp)
    for r in range(world):
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm), (r, res[r]["grad_norm"], ref_norm)
        got = torch.from_numpy(res[r]["full"])
        assert got.shape == ref_flat.shape
        assert torch.allclose(got, ref_flat.float(), atol=3e-4), (r, (got - ref_flat.float()).abs().max())
        assert torch.allclose(torch.from_numpy(res[r]["log_probs"]), rows[r // (tp * pp)], atol=1e-4), r


def test_expert_parallel_with_expert_tensor_parallel_matches_unsharded():
    """Four ranks: two data-parallel replicas that split the experts between them, each replica two tensor-parallel ranks
    that split every expert's width (and the attention heads). Tokens travel to the owner of their expert inside each
    tensor-parallel rank's own expert-parallel group; the re-assembled full model, the gradient norm and the log-probs
    equal one process."""
    ref_norm, ref_lp, ref_flat = _reference("tiny-moe")
    res = _run(4, 2, 1, ep=2, preset="tiny-moe")
    rows = ref_lp.chunk(2)
    for r in range(4):
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm), (r, res[r]["grad_norm"], ref_norm)
        got = torch.from_numpy(res[r]["full"])
        assert got.shape == ref_flat.shape
        assert torch.allclose(got, ref_flat.float(), atol=3e-4), (r, (got - ref_flat.float()).abs().max())
        assert torch.allclose(torch.from_numpy(res[r]["log_probs"]), rows[r // 2], atol=1e-4), r


def test_expert_parallel_engine_matches_unsharded():
    """Two ranks, each with half of the experts and half of the batch: same gradient norm, same updated full model and the
    same log-probs as one process that holds every expert and sees the whole batch."""
    ref_norm, ref_lp, ref_flat = _reference("tiny-moe")
    res = _run(2, 1, 1, ep=2, preset="tiny-moe")
    rows = ref_lp.chunk(2)
    for r in range(2):
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm), (r, res[r]["grad_norm"], ref_norm)
        got = torch.from_numpy(res[r]["full"])
        assert got.shape == ref_flat.shape
        assert torch.allclose(got, ref_flat.float(), atol=3e-4), (r, (got - ref_flat.float()).abs().max())
        assert torch.allclose(torch.from_numpy(res[r]["log_probs"]), rows[r], atol=1e-4), r


def _ppo_proc(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      VERL_ENGINE_DEVICE="cpu")
    try:
        from verl_b200.trainer.main_ppo import main

        t = main(['actor@actor_rollout_ref.actor=megatron_actor', 'actor_rollout_ref.actor.megatron.tensor_model_parallel_size=2',
                  'data.train_batch_size=4', 'data.max_prompt_length=16', 'data.max_response_length=12', 'data.synthetic.num_prompts=16',
                  'data.synthetic.prompt_length=16', 'data.synthetic.vocab_high=512', 'actor_rollout_ref.model.path=tiny-qwen2',
                  'actor_rollout_ref.rollout.n=2', 'actor_rollout_ref.actor.ppo_mini_batch_size=4',
                  'actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4', 'actor_rollout_ref.actor.use_kl_loss=true',
                  'actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8', 'actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=8',
                  'actor_rollout_ref.rollout.tensor_model_parallel_size=2', 'algorithm.adv_estimator=grpo',
                  'reward_model.reward_manager=token_rule', 'trainer.n_gpus_per_node=2', 'trainer.total_epochs=2',
                  'trainer.total_training_steps=2', 'trainer.device=cpu', 'trainer.val_before_train=false',
                  'actor_rollout_ref.rollout.max_num_seqs=8', 'actor_rollout_ref.rollout.block_size=8', 'trainer.resume_mode=disable',
                  'trainer.worker_group=spmd', 'trainer.logger=[]'])
        b = t.last_batch.batch
        diff = (torch.exp(b["rollout_log_probs"]) - torch.exp(b["old_log_probs"])).abs()[b["response_mask"].bool()].max().item()
        q.put((rank, {"steps": t.global_steps, "adv_shape": tuple(b["advantages"].shape), "prob_diff": diff,
                      "resp": b["responses"].numpy()}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_grpo_end_to_end_with_tensor_parallel_actor_and_rollout():
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_ppo_proc, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=400) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    for r in (0, 1):
        assert "error" not in res[r], res[r]["error"]
        assert res[r]["steps"] == 3 and res[r]["adv_shape"] == (8, 12)
        assert res[r]["prob_diff"] < 1e-3  # TP-sharded trainer and TP rollout on gathered weights agree on token probabilities
    assert (res[0]["resp"] == res[1]["resp"]).all()  # one replica: both ranks hold the same batch


def _ppo_ep_proc(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      VERL_ENGINE_DEVICE="cpu")
    try:
        from verl_b200.trainer.main_ppo import main

        t = main(['actor@actor_rollout_ref.actor=megatron_actor', 'actor_rollout_ref.actor.megatron.expert_model_parallel_size=2',
                  'data.train_batch_size=4', 'data.max_prompt_length=16', 'data.max_response_length=12', 'data.synthetic.num_prompts=16',
                  'data.synthetic.prompt_length=16', 'data.synthetic.vocab_high=512', 'actor_rollout_ref.model.path=tiny-moe',
                  'actor_rollout_ref.rollout.n=2', 'actor_rollout_ref.actor.ppo_mini_batch_size=4',
                  'actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4', 'actor_rollout_ref.actor.use_kl_loss=true',
                  'actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8', 'actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=8',
                  'algorithm.adv_estimator=grpo', 'reward_model.reward_manager=token_rule', 'trainer.n_gpus_per_node=2',
                  'trainer.total_epochs=2', 'trainer.total_training_steps=2', 'trainer.device=cpu', 'trainer.val_before_train=false',
                  'actor_rollout_ref.rollout.max_num_seqs=8', 'actor_rollout_ref.rollout.block_size=8', 'trainer.resume_mode=disable',
                  'trainer.worker_group=spmd', 'trainer.logger=[]'])
        b = t.last_batch.batch
        diff = (torch.exp(b["rollout_log_probs"]) - torch.exp(b["old_log_probs"])).abs()[b["response_mask"].bool()].max().item()
        q.put((rank, {"steps": t.global_steps, "adv_shape": tuple(b["advantages"].shape), "prob_diff": diff,
                      "resp": b["responses"].numpy()}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_grpo_end_to_end_with_expert_parallel_actor():
    """Mixture-of-experts actor with the experts split over the two data-parallel ranks; the rollout engine of each rank
    runs on the full model gathered from the shards after every update."""
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_ppo_ep_proc, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=400) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    for r in (0, 1):
        assert "error" not in res[r], res[r]["error"]
        assert res[r]["steps"] == 3 and res[r]["adv_shape"] == (4, 12)   # two ranks x (2 prompts x 2 samples)
        assert res[r]["prob_diff"] < 1e-3  # expert-sharded trainer and full-model rollout agree on token probabilities
    assert not (res[0]["resp"] == res[1]["resp"]).all()  # data parallel: the ranks hold different prompts


def _ppo_critic_proc(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      VERL_ENGINE_DEVICE="cpu")
    try:
        from verl_b200.trainer.main_ppo import main

        t = main(['actor@actor_rollout_ref.actor=megatron_actor', 'actor_rollout_ref.actor.megatron.pipeline_model_parallel_size=2',
                  'critic@critic=megatron_critic', 'critic.megatron.pipeline_model_parallel_size=2', 'critic.model.path=tiny-llama',
                  'critic.ppo_micro_batch_size_per_gpu=4', 'critic.ppo_mini_batch_size=4',
                  'data.train_batch_size=4', 'data.max_prompt_length=16', 'data.max_response_length=12', 'data.synthetic.num_prompts=16',
                  'data.synthetic.prompt_length=16', 'data.synthetic.vocab_high=512', 'actor_rollout_ref.model.path=tiny-llama',
                  'actor_rollout_ref.rollout.n=1', 'actor_rollout_ref.actor.ppo_mini_batch_size=4',
                  'actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=2', 'actor_rollout_ref.actor.use_kl_loss=false',
                  'actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=2', 'actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=2',
                  'actor_rollout_ref.rollout.tensor_model_parallel_size=1', 'algorithm.adv_estimator=gae',
                  'reward_model.reward_manager=token_rule', 'trainer.n_gpus_per_node=2', 'trainer.total_epochs=2',
                  'trainer.total_training_steps=2', 'trainer.device=cpu', 'trainer.val_before_train=false',
                  'actor_rollout_ref.rollout.max_num_seqs=8', 'actor_rollout_ref.rollout.block_size=8', 'trainer.resume_mode=disable',
                  'trainer.worker_group=spmd', 'trainer.logger=[]'])
        b = t.last_batch.batch
        q.put((rank, {"steps": t.global_steps, "keys": sorted(b.keys()), "resp": b["responses"].numpy(), "values": b["values"].numpy(),
                      "critic": type(t.critic_wg.worker.engine).__name__, "pp": t.critic_wg.worker.engine.topo.pp}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_ppo_with_critic_under_pipeline_parallelism():
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_ppo_critic_proc, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=400) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    for r in (0, 1):
        assert "error" not in res[r], res[r]["error"]
        assert res[r]["steps"] == 3 and "values" in res[r]["keys"] and "returns" in res[r]["keys"]
        assert res[r]["critic"] == "ModelParallelEngineWithValueHead" and res[r]["pp"] == 2
    assert (res[0]["resp"] == res[1]["resp"]).all() and abs(res[0]["values"] - res[1]["values"]).max() < 1e-5
