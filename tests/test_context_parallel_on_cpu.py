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


def test_dynamic_cp_scheduler_packs_rows_into_aligned_groups():
    from verl_b200.utils.dynamic_cp_scheduler import DynamicCPScheduler, required_group_size

    assert [required_group_size(n, 100, 8) for n in (1, 100, 101, 200, 201, 799)] == [1, 1, 2, 2, 4, 8]
    with pytest.raises(ValueError):
        required_group_size(801, 100, 8)
    with pytest.raises(ValueError):
        DynamicCPScheduler(100, 6)
    lens = [790, 30, 410, 95, 180, 60, 20, 399, 100, 5, 150, 77]
    sch = DynamicCPScheduler(100, 8)
    plan = sch.schedule(lens)
    seen = []
    for mb in plan:
        assert len(mb) == 8
        for r, a in enumerate(mb):
            if not a.rows:
                continue
            assert a.start % a.size == 0 and a.start <= r < a.start + a.size           # aligned window that contains the rank
            assert all(mb[q].rows == a.rows and mb[q].size == a.size for q in range(a.start, a.start + a.size))
            assert all(-(-lens[i] // a.size) <= 100 for i in a.rows)
            if r == a.start:
                seen += a.rows
    assert sorted(seen) == list(range(len(lens)))                                       # every row exactly once
    loads = sch.loads(lens, plan)
    assert all(x <= 100 + 1e-9 for mb in loads for x in mb)
    assert len(plan) <= 4                                                               # 2516 tokens, 800 per micro-batch at best
    # one long row: the whole block; only short rows: single ranks, spread over the block
    assert [a.size for a in DynamicCPScheduler(100, 4).schedule([400])[0]] == [4] * 4
    p = DynamicCPScheduler(100, 4).schedule([50, 50, 50, 50])
    assert len(p) == 1 and sorted(a.rows[0] for a in p[0]) == [0, 1, 2, 3] and all(a.size == 1 for a in p[0])


def _ragged_data():
    """Rows of 24, 17, 12 and 24 valid tokens (right-padded responses), so that the rows need different group sizes."""
    data = _data()
    am = data["attention_mask"].clone()
    am[1, 20:] = 0
    am[2, 12:] = 0
    data["attention_mask"] = am
    data["response_mask"] = am[:, -data["responses"].shape[1]:].clone()
    return data


def _dyn_proc(rank, world, port, cp, q):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                          VERL_ENGINE_DEVICE="cpu")
        from functools import partial

        from verl_b200.models import get_preset
        from verl_b200.utils.distributed import initialize_global_process_group
        from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
        from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
        from verl_b200.workers.utils.losses import sft_loss

        initialize_global_process_group()
        ec = FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=2, context_parallel_size=cp, dynamic_context_parallel=True,
                              max_seqlen_per_dp_cp_rank=12)
        eng = NativeEngineWithLMHead(get_preset("tiny-llama"), ec, OptimizerConfig(lr=1e-2, clip_grad=0.05))
        eng.initialize()
        dp = world // cp
        data = _ragged_data()
        shard = {k: v.chunk(dp)[rank // cp] for k, v in data.items()}
        out = eng.train_batch(dict(shard), partial(sft_loss, None))
        sizes = sorted({a.size for mb in eng.last_dcp_plan for a in mb if a.rows})
        lp = eng.infer_batch(dict(shard))["model_output"]["log_probs"]
        q.put((rank, {"grad_norm": float(out["metrics"]["grad_norm"]), "flat": eng.params.flat.float().numpy(), "lp": lp.float().numpy(),
                      "sizes": sizes, "restored": eng.sp_size == cp}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


@pytest.mark.parametrize("world,cp", [(4, 4), (2, 2)])
def test_dynamic_context_parallel_matches_single_rank(world, cp):
    """A group size per row (rows of 24, 17, 12 and 24 tokens with 12 tokens per rank: groups of 2, 2, 1 and 2 ranks) gives
    the update and the log-probs of one rank that holds everything."""
    import torch.multiprocessing as mp

    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from functools import partial

    from verl_b200.models import get_preset
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.utils.losses import sft_loss

    data = _ragged_data()
    ref = NativeEngineWithLMHead(get_preset("tiny-llama"), FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=2), OptimizerConfig(lr=1e-2, clip_grad=0.05))
    ref.initialize()
    ref_norm = float(ref.train_batch(dict(data), partial(sft_loss, None))["metrics"]["grad_norm"])
    ref_lp = ref.infer_batch(dict(data))["model_output"]["log_probs"]
    ref_flat = ref.params.flat.clone()

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_dyn_proc, args=(r, world, port, cp, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(world))
    for p in ps:
        p.join(timeout=30)
    m = data["attention_mask"][:, -ref_lp.shape[1]:].bool()
    for r in range(world):
        assert "error" not in res[r], res[r]["error"]
        assert res[r]["restored"] and len(res[r]["sizes"]) >= 2, res[r]["sizes"]           # more than one group size was in use
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm), (r, res[r]["grad_norm"], ref_norm)
        n = min(ref_flat.numel(), res[r]["flat"].size)     # the flat buffer is padded to a multiple of the world size
        assert torch.allclose(torch.from_numpy(res[r]["flat"])[:n], ref_flat.float()[:n], atol=3e-4), r
        assert torch.allclose(torch.from_numpy(res[r]["lp"])[m], ref_lp[m], atol=1e-4), r
