"""Context parallelism on gloo: ranks that split the tokens of the same micro-batches and gather keys / values around
attention reproduce the single-rank update, also where the group size does not divide the KV heads."""
import os
import socket

import pytest
import torch

from tests.test_model_parallel_engine_on_cpu import _data, _reference


def test_query_slice_attention_matches_full_attention():
    from verl_b200.ops import functional as F

    torch.manual_seed(0)
    cu = torch.tensor([0, 5, 14, 17], dtype=torch.int32)
    T = 17
    q, k, v, g = torch.randn(T, 4, 16), torch.randn(T, 2, 16), torch.randn(T, 2, 16), torch.randn(T, 4, 16)
    ref, _ = F.attention_varlen(q, k, v, cu, 9)
    dq, dk, dv = F.attention_varlen_bwd(g, q, k, v, ref, None, cu, 9)
    dks, dvs = torch.zeros_like(k), torch.zeros_like(v)
    for lo, hi in ((0, 6), (6, 12), (12, 17)):          # slices that cut through sequences
        o = F.attention_query_slice(q[lo:hi], k, v, cu, lo)
        assert torch.allclose(o, ref[lo:hi], atol=1e-6)
        a, b, c = F.attention_query_slice_bwd(g[lo:hi], q[lo:hi], k, v, cu, lo)
        assert torch.allclose(a, dq[lo:hi], atol=1e-5)
        dks += b
        dvs += c
    assert torch.allclose(dks, dk, atol=1e-5) and torch.allclose(dvs, dv, atol=1e-5)


def _proc(rank, world, port, cp, q, mode="zigzag"):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                          VERL_ENGINE_DEVICE="cpu")
        from functools import partial

        from verl_b200.models import get_preset
        from verl_b200.models.decoder import ContextParallel
        from verl_b200.utils.distributed import initialize_global_process_group
        from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
        from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
        from verl_b200.workers.utils.losses import sft_loss

        initialize_global_process_group()
        ec = FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=2, context_parallel_size=cp, context_parallel_mode=mode)
        eng = NativeEngineWithLMHead(get_preset("tiny-llama"), ec, OptimizerConfig(lr=1e-2, clip_grad=0.05))
        eng.initialize()
        assert isinstance(eng.model.sp, ContextParallel) and eng.model.sp.zigzag == (mode == "zigzag")
        dp = world // cp
        shard = {k: v.chunk(dp)[rank // cp] for k, v in _data().items()}
        out = eng.train_batch(dict(shard), partial(sft_loss, None))
        lp = eng.infer_batch(dict(shard))["model_output"]["log_probs"]
        q.put((rank, {"grad_norm": float(out["metrics"]["grad_norm"]), "flat": eng.params.flat.float().numpy(), "lp": lp.float().numpy()}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


@pytest.mark.parametrize("world,cp,mode", [(3, 3, "zigzag"), (2, 2, "contiguous")])
def test_context_parallel_matches_single_rank(world, cp, mode):
    import torch.multiprocessing as mp

    ref_norm, ref_lp, ref_flat = _reference()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_proc, args=(r, world, port, cp, q, mode)) for r in range(world)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(world))
    for p in ps:
        p.join(timeout=30)
    rows = ref_lp.chunk(world // cp)
    for r in range(world):
        assert "error" not in res[r], res[r]["error"]
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm), (world, r, res[r]["grad_norm"], ref_norm)
        n = ref_flat.numel()
        assert torch.allclose(torch.from_numpy(res[r]["flat"])[:n], ref_flat.float(), atol=3e-4)
        assert torch.allclose(torch.from_numpy(res[r]["lp"]), rows[r // cp], atol=1e-4)


def _ppo_proc(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      VERL_ENGINE_DEVICE="cpu")
    try:
        from verl_b200.trainer.main_ppo import main

        t = main(['actor_rollout_ref.actor.fsdp_config.context_parallel_size=2', 'data.train_batch_size=4', 'data.max_prompt_length=16',
                  'data.max_response_length=12', 'data.synthetic.num_prompts=16', 'data.synthetic.prompt_length=16',
                  'data.synthetic.vocab_high=512', 'actor_rollout_ref.model.path=tiny-qwen2', 'actor_rollout_ref.rollout.n=2',
                  'actor_rollout_ref.actor.ppo_mini_batch_size=4', 'actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4',
                  'actor_rollout_ref.actor.use_kl_loss=true', 'actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8',
                  'actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=8', 'actor_rollout_ref.rollout.tensor_model_parallel_size=1',
                  'algorithm.adv_estimator=grpo', 'reward_model.reward_manager=token_rule', 'trainer.n_gpus_per_node=2',
                  'trainer.total_epochs=2', 'trainer.total_training_steps=2', 'trainer.device=cpu', 'trainer.val_before_train=false',
                  'actor_rollout_ref.rollout.max_num_seqs=8', 'actor_rollout_ref.rollout.block_size=8', 'trainer.resume_mode=disable',
                  'trainer.worker_group=spmd', 'trainer.logger=[]'])
        b = t.last_batch.batch
        diff = (torch.exp(b["rollout_log_probs"]) - torch.exp(b["old_log_probs"])).abs()[b["response_mask"].bool()].max().item()
        eng = t.actor_rollout_wg.worker.actor
        q.put((rank, {"steps": t.global_steps, "shape": tuple(b["advantages"].shape), "prob_diff": diff, "resp": b["responses"].numpy(),
                      "cp": eng.cp_size, "kind": type(eng.model.sp).__name__}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_grpo_end_to_end_with_context_parallel_actor():
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
        assert res[r]["steps"] == 3 and res[r]["shape"] == (8, 12) and res[r]["cp"] == 2 and res[r]["kind"] == "ContextParallel"
        assert res[r]["prob_diff"] < 1e-3
    assert (res[0]["resp"] == res[1]["resp"]).all()


def _tp_cp_proc(rank, world, port, q):
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
        eng = EngineRegistry.new("language_model", "megatron", model_config=get_preset("tiny-llama"),
                                 engine_config=McoreEngineConfig(seed=7, micro_batch_size_per_gpu=2, tensor_model_parallel_size=2,
                                                                 context_parallel_size=2),
                                 optimizer_config=OptimizerConfig(lr=1e-2, clip_grad=0.05))
        eng.initialize()
        out = eng.train_batch(dict(_data()), partial(sft_loss, None))
        q.put((rank, {"grad_norm": float(out["metrics"]["grad_norm"]), "kinds": (type(eng.model.sp).__name__, eng.model.tsp is None)}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_tensor_parallel_times_context_parallel():
    import torch.multiprocessing as mp

    from verl_b200.models import get_preset
    from verl_b200.workers.config import McoreEngineConfig
    from verl_b200.workers.engine.base import EngineRegistry

    ref_norm, _, _ = _reference()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_tp_cp_proc, args=(r, 4, port, q)) for r in range(4)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(4))
    for p in ps:
        p.join(timeout=30)
    for r in range(4):
        assert "error" not in res[r], res[r]["error"]
        assert res[r]["kinds"] == ("ContextParallel", True)
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm)
    with pytest.raises(NotImplementedError, match="pipeline"):
        EngineRegistry.new("language_model", "megatron", model_config=get_preset("tiny-llama"),
                           engine_config=McoreEngineConfig(pipeline_model_parallel_size=2, context_parallel_size=2), optimizer_config=None)


def test_zigzag_layout_bookkeeping():
    from verl_b200.models.decoder import ContextParallel

    total, size = 24, 3
    seen = []
    for r in range(size):
        cp = ContextParallel(None, r, size)
        assert cp.pad_multiple() == 6 and cp.chunks(total) == [(4 * r, 4 * r + 4), (4 * (5 - r), 4 * (5 - r) + 4)]
        rows = cp.local_rows(total)
        seen.append(rows)
        pos = torch.tensor([0, 5, 9, 14, 19, 23])
        mine, local = cp.local_of(pos, total)
        assert torch.equal(rows[local], pos[mine])
    assert torch.equal(torch.cat(seen).sort().values, torch.arange(total))         # every token has exactly one owner
    # rank-major gathered rows -> stream order and back
    cp = ContextParallel(None, 1, size)
    gathered = torch.cat(seen)                                                    # what an all-gather of the rows delivers
    order = cp._stream_order(total, "cpu")
    assert torch.equal(gathered[order], torch.arange(total))
    flat = ContextParallel(None, 1, size, zigzag=False)
    assert flat.pad_multiple() == 3 and flat.chunks(total) == [(8, 16)] and flat._stream_order(total, "cpu") is None
