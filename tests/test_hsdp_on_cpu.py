"""Hybrid sharding (fsdp_size): shards inside blocks of ranks, replicas across blocks; equals the unsharded engine."""
import os
import socket

import pytest
import torch


def _data(seed=0, b=8, L=24, R=16, V=500):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(3, V, (b, L), generator=g)
    am = torch.ones_like(ids)
    am[1, :3] = 0
    return {"input_ids": ids, "attention_mask": am, "responses": ids[:, -R:], "response_mask": am[:, -R:]}


def _proc(rank, world, port, fsdp_size, tmp, q):
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
        mk = lambda: NativeEngineWithLMHead(get_preset("tiny-llama"), FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=2, fsdp_size=fsdp_size),
                                            OptimizerConfig(lr=1e-2, clip_grad=0.05))
        eng = mk()
        eng.initialize()
        shard = {k: v.chunk(world)[rank] for k, v in _data().items()}
        out = eng.train_batch(dict(shard), partial(sft_loss, None))
        res = {"grad_norm": float(out["metrics"]["grad_norm"]), "flat": eng.params.flat.float().numpy(),
               "layout": (eng.sh_world, eng.sh_rank, eng.rep_world, eng.rep_rank), "master_numel": eng.master.numel()}
        eng.save_checkpoint(tmp)
        eng2 = mk()
        eng2.initialize()
        eng2.load_checkpoint(tmp)
        res["reload_equal"] = bool(torch.equal(eng2.params.flat, eng.params.flat) and torch.equal(eng2.exp_avg, eng.exp_avg))
        res["files"] = sorted(f for f in os.listdir(tmp) if f.startswith("model_"))
        q.put((rank, res))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


@pytest.mark.parametrize("fsdp_size", [2, 1])
def test_hybrid_sharding_matches_unsharded(fsdp_size, tmp_path):
    import torch.multiprocessing as mp
    from functools import partial

    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from verl_b200.models import get_preset
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.utils.losses import sft_loss

    ref = NativeEngineWithLMHead(get_preset("tiny-llama"), FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=2), OptimizerConfig(lr=1e-2, clip_grad=0.05))
    ref.initialize()
    ref_norm = float(ref.train_batch(dict(_data()), partial(sft_loss, None))["metrics"]["grad_norm"])
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_proc, args=(r, 4, port, fsdp_size, str(tmp_path), q)) for r in range(4)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(4))
    for p in ps:
        p.join(timeout=30)
    for r in range(4):
        assert "error" not in res[r], res[r]["error"]
        assert res[r]["layout"] == (fsdp_size, r % fsdp_size, 4 // fsdp_size, r // fsdp_size)
        assert 0 <= res[r]["master_numel"] * fsdp_size - ref.params.numel < 1024   # one shard per block member (plus padding)
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm), (r, res[r]["grad_norm"], ref_norm)
        got = torch.from_numpy(res[r]["flat"])[: ref.params.numel]
        assert ((got - ref.params.flat.float()).abs() > 3e-4).float().mean() < 1e-3
        assert res[r]["reload_equal"]
        assert res[r]["files"] == [f"model_world_size_{fsdp_size}_rank_{i}.pt" for i in range(fsdp_size)]
    if fsdp_size == 2:
        # a checkpoint written by two shards loads into one: every range is rebuilt from the files that overlap it
        one = NativeEngineWithLMHead(get_preset("tiny-llama"), FSDPEngineConfig(seed=11, micro_batch_size_per_gpu=2), OptimizerConfig(lr=1e-2, clip_grad=0.05))
        one.initialize()
        one.load_checkpoint(str(tmp_path))
        n = one.params.numel
        assert torch.equal(one.params.flat.float()[:n], torch.from_numpy(res[0]["flat"])[:n])
        assert one.opt_step_count == 1 and float(one.exp_avg.abs().sum()) > 0
        assert abs(float(one.exp_avg.double().pow(2).sum()) - float(ref.exp_avg.double().pow(2).sum())) < 1e-4 * float(ref.exp_avg.double().pow(2).sum()) + 1e-12
        # a shard file that is gone is an error, not a silent fresh start
        os.remove(os.path.join(str(tmp_path), "optim_world_size_2_rank_1.pt"))
        with pytest.raises(FileNotFoundError, match="world size 2"):
            one.load_checkpoint(str(tmp_path))


def test_checkpoint_load_refuses_missing_files_and_rotates(tmp_path):
    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from verl_b200.models import get_preset
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead

    eng = NativeEngineWithLMHead(get_preset("tiny-llama"), FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=2), OptimizerConfig(lr=1e-2))
    eng.initialize()
    with pytest.raises(FileNotFoundError):
        eng.load_checkpoint(str(tmp_path / "nowhere"))
    dirs = [str(tmp_path / f"global_step_{i}" / "actor") for i in range(3)]
    for d in dirs:
        eng.save_checkpoint(d, max_ckpt_to_keep=2)
    assert not os.path.isdir(dirs[0]) and os.path.isdir(dirs[1]) and os.path.isdir(dirs[2])
    os.remove(os.path.join(dirs[2], "model_world_size_1_rank_0.pt"))
    with pytest.raises(FileNotFoundError, match="model_world_size_1_rank_0"):
        eng.load_checkpoint(dirs[2])
    eng.load_checkpoint(dirs[1])
