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


def _proc(rank, world, port, tp, pp, q):
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
        ec = McoreEngineConfig(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp, seed=7, micro_batch_size_per_gpu=2)
        eng = EngineRegistry.new("language_model", "megatron", get_preset("tiny-llama"), ec, OptimizerConfig(lr=1e-2, clip_grad=0.05), device="cpu")
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


def _run(world, tp, pp):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_proc, args=(r, world, port, tp, pp, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(world))
    for p in ps:
        p.join(timeout=30)
    for r in range(world):
        assert "error" not in res[r], res[r]["error"]
    return res


def _reference():
    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from functools import partial

    from verl_b200.models import get_preset
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.utils.losses import sft_loss

    eng = NativeEngineWithLMHead(get_preset("tiny-llama"), FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=2), OptimizerConfig(lr=1e-2, clip_grad=0.05))
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
