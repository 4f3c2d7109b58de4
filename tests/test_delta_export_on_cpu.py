"""Sparse export of an optimizer step from model-parallel shards: the records of all ranks, applied to the HF-named tensors
of the previous step, give the HF-named tensors of the new step."""
import os
import socket

import pytest
import torch


def test_full_positions_arithmetic():
    from verl_b200.parallel.model_parallel import ShardMap
    from verl_b200.workers.engine.mp.delta_export import full_positions

    full = torch.arange(12 * 6).view(12, 6)
    # column slice of rank 1 of 2
    loc = full[:, 3:6].contiguous()
    idx = torch.tensor([0, 4, 17])
    pos = full_positions(ShardMap("a", "a", "cols"), idx, tuple(loc.shape), (12, 6), 2, 1)
    assert torch.equal(full.view(-1)[pos], loc.view(-1)[idx])
    # stacked row blocks (8 | 2 | 2), each cut in two: rank 1 holds rows 4..8, 9, 11
    m = ShardMap("a", "a", "rows", (8, 2, 2))
    loc = torch.cat([full[4:8], full[9:10], full[11:12]])
    idx = torch.arange(loc.numel())
    pos = full_positions(m, idx, tuple(loc.shape), (12, 6), 2, 1)
    assert torch.equal(full.view(-1)[pos], loc.view(-1))
    # experts: rank 1 of 2 holds the second half of dim 0
    fe = torch.arange(4 * 3 * 5).view(4, 3, 5)
    pos = full_positions(ShardMap("e", "e", "experts"), torch.tensor([0, 7, 29]), (2, 3, 5), (4, 3, 5), 1, 0, 2, 1)
    assert torch.equal(fe.view(-1)[pos], fe[2:].reshape(-1)[torch.tensor([0, 7, 29])])


def _proc(rank, world, port, model, kw, q):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                          VERL_ENGINE_DEVICE="cpu")
        from functools import partial

        import torch.distributed as dist

        from tests.test_model_parallel_engine_on_cpu import _data
        from verl_b200.models import get_preset
        from verl_b200.utils.distributed import initialize_global_process_group
        from verl_b200.workers.config import McoreEngineConfig, OptimizerConfig
        from verl_b200.workers.engine.base import EngineRegistry
        from verl_b200.workers.engine.mp.delta_export import ShardDeltaExporter, apply_hf_delta
        from verl_b200.workers.utils.losses import sft_loss

        initialize_global_process_group()
        eng = EngineRegistry.new("language_model", "megatron", model_config=get_preset(model),
                                 engine_config=McoreEngineConfig(seed=7, micro_batch_size_per_gpu=2, **kw),
                                 optimizer_config=OptimizerConfig(lr=1e-2, clip_grad=1.0))
        eng.initialize()
        before = eng.gather_full_params(torch.float32).hf_state_dict(clone=True)
        exp = ShardDeltaExporter(eng)
        assert exp.export() == []                                      # nothing changed yet
        data = _data()
        dp = eng.world
        shard = {k: v.chunk(dp)[eng.rank] for k, v in data.items()}
        eng.train_batch(dict(shard), partial(sft_loss, None))
        frac = exp.changed_fraction()
        recs = exp.export()
        box = [None] * world
        dist.all_gather_object(box, (rank, eng.rank, recs))
        after = eng.gather_full_params(torch.float32).hf_state_dict(clone=True)
        patched = {k: v.clone() for k, v in before.items()}
        total = 0
        for _, dp_rank, r in box:
            if dp_rank == 0 or model == "tiny-moe":                    # one data-parallel replica (expert shards differ per rank)
                total += apply_hf_delta(patched, r)
        worst = max(float((patched[k] - after[k]).abs().max()) for k in after)
        changed = sum(int((before[k] != after[k]).sum()) for k in after)
        q.put((rank, {"worst": worst, "total": total, "changed": changed, "frac": frac, "again": len(exp.export())}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


@pytest.mark.parametrize("model,world,kw", [
    ("tiny-qwen2", 4, dict(tensor_model_parallel_size=2, pipeline_model_parallel_size=2)),
    ("tiny-moe", 2, dict(expert_model_parallel_size=2)),
])
def test_exported_records_rebuild_the_new_weights(model, world, kw):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_proc, args=(r, world, port, model, kw, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(world))
    for p in ps:
        p.join(timeout=30)
    for r in range(world):
        assert "error" not in res[r], res[r]["error"]
        assert res[r]["worst"] == 0.0, res[r]
        assert res[r]["total"] >= res[r]["changed"] > 0 and 0 < res[r]["frac"] <= 1 and res[r]["again"] == 0
