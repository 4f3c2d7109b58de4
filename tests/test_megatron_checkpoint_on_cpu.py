"""Model-parallel checkpoints in layout schema v2: every model-parallel rank writes its own shard directory, the manifest
comes last, a fresh job of the same layout resumes bit-exactly, the merger rebuilds the HF model, incomplete or
flat-layout directories are refused, and the migration converts a flat directory in place."""
import json
import os
import shutil
import socket

import pytest
import torch


def _data(seed=0, b=4, L=24, R=16, V=500):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(3, V, (b, L), generator=g)
    am = torch.ones_like(ids)
    return {"input_ids": ids, "attention_mask": am, "responses": ids[:, -R:], "response_mask": am[:, -R:]}


def _proc(rank, world, port, tp, pp, ep, preset, tmp, q):
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
        ckpt_cfg = type("C", (), {"save_contents": ["model", "optimizer", "extra", "hf_model"], "load_contents": ["model", "optimizer", "extra"]})()

        def make(seed):
            ec = McoreEngineConfig(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp, expert_model_parallel_size=ep, seed=seed,
                                   micro_batch_size_per_gpu=2)
            e = EngineRegistry.new("language_model", "megatron", get_preset(preset), ec, OptimizerConfig(lr=1e-2, clip_grad=0.05),
                                   checkpoint_config=ckpt_cfg, device="cpu")
            e.initialize()
            return e

        eng = make(7)
        shard = {k: v.chunk(eng.topo.dp)[eng.topo.dp_rank] for k, v in _data().items()}
        eng.train_batch(dict(shard), partial(sft_loss, None))
        d = os.path.join(tmp, "global_step_1", "actor")
        eng.save_checkpoint(d, global_step=1)
        full = eng.gather_full_params()
        res = {"full": full.flat.float().numpy()}
        if rank == 0:
            torch.save({k: v.clone() for k, v in full.hf_views()}, os.path.join(tmp, "ref.pt"))
        # a fresh job of the same layout resumes: same weights, same next step
        eng2 = make(123)
        eng2.load_checkpoint(d)
        res["resume_equal"] = bool(torch.equal(eng2.gather_full_params().flat, full.flat) and torch.equal(eng2.exp_avg, eng.exp_avg)
                                   and eng2.opt_step_count == eng.opt_step_count)
        n1 = float(eng.train_batch(dict(shard), partial(sft_loss, None))["metrics"]["grad_norm"])
        n2 = float(eng2.train_batch(dict(shard), partial(sft_loss, None))["metrics"]["grad_norm"])
        res["next_step_equal"] = abs(n1 - n2) < 1e-6 * max(1.0, n1) and bool(torch.equal(eng2.params.flat, eng.params.flat))
        q.put((rank, res))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


@pytest.mark.parametrize("tp,pp,ep,preset", [(2, 2, 1, "tiny-llama"), (1, 1, 2, "tiny-moe")])
def test_layout_v2_round_trip_and_merge(tp, pp, ep, preset, tmp_path):
    import torch.multiprocessing as mp

    world = max(tp * pp, ep)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_proc, args=(r, world, port, tp, pp, ep, preset, str(tmp_path), q)) for r in range(world)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(world))
    for p in ps:
        p.join(timeout=30)
    for r in range(world):
        assert "error" not in res[r], res[r]["error"]
        assert res[r]["resume_equal"] and res[r]["next_step_equal"], (r, res[r]["resume_equal"], res[r]["next_step_equal"])
    d = tmp_path / "global_step_1" / "actor"
    man = json.loads((d / "ckpt_contents.json").read_text())
    assert man["schema_version"] == 2 and man["global_step"] == 1 and man["role"] == "actor"
    assert man["backend"]["tensor_parallel"] == tp and man["backend"]["pipeline_parallel"] == pp and man["backend"]["expert_parallel"] == ep
    assert {"model", "optimizer", "rng_state", "hf_config", "hf_model", "transformer_config", "lr_scheduler"} <= set(man["contents"])
    dirs = sorted(os.listdir(d / "model" / "dist_ckpt"))
    want = [f"mp_rank_{t:02d}_{p:03d}" for p in range(pp) for t in range(tp)] if ep == 1 else [f"mp_rank_00_000_{e:03d}" for e in range(ep)]
    assert dirs == sorted(want)
    assert (d / "transformer_config.json").exists() and (d / "model" / "huggingface" / "config.json").exists()
    assert sorted(os.listdir(d / "optimizer" / "dist_ckpt")) == sorted(want)
    # the merger rebuilds the HF tensors from the shards
    from verl_b200.model_merger.base_model_merger import ModelMergerConfig
    from verl_b200.model_merger.megatron_model_merger import MegatronModelMerger

    merged = MegatronModelMerger(ModelMergerConfig(operation="merge", backend="megatron", local_dir=str(d), target_dir=str(d / "out"),
                                                   hf_model_config_path=str(d / "model" / "huggingface"))).merge_state_dict()
    ref = torch.load(tmp_path / "ref.pt")
    for k, v in ref.items():
        if k == "lm_head.weight" and k not in merged:
            continue
        assert torch.allclose(merged[k].float(), v.float(), atol=1e-2), k
    assert len(merged) >= len(ref) - 1


def test_incomplete_and_flat_layouts_are_refused_and_migrated(tmp_path):
    from verl_b200.utils.checkpoint.megatron_checkpoint_manager import MegatronCheckpointManager, migrate_layout

    class Topo:
        tp_rank = pp_rank = dp_rank = ep_rank = 0
        tp = pp = dp = ep = 1

    class Eng:
        topo, forward_only, value_head = Topo(), True, False

    mgr = MegatronCheckpointManager(Eng(), checkpoint_config=type("C", (), {"save_contents": ["model"], "load_contents": ["model"]})())
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(FileNotFoundError, match="manifest is written last"):
        mgr.load_checkpoint(str(empty))
    flat = tmp_path / "actor"
    (flat / "mp_rank_00_000").mkdir(parents=True)
    torch.save({"w": torch.ones(2)}, flat / "mp_rank_00_000" / "model.pt")
    torch.save({"master": torch.ones(2)}, flat / "mp_rank_00_000" / "optim_dp0.pt")
    (flat / "huggingface").mkdir()
    (flat / "huggingface" / "config.json").write_text("{}")
    with pytest.raises(RuntimeError, match="flat layout"):
        mgr.load_checkpoint(str(flat))
    man = migrate_layout(str(flat))
    assert man["schema_version"] == 2 and man["contents"]["model"]["path"] == "model/dist_ckpt"
    assert (flat / "model" / "dist_ckpt" / "mp_rank_00_000" / "model.pt").exists()
    assert (flat / "optimizer" / "dist_ckpt" / "mp_rank_00_000" / "optim_dp0.pt").exists()
    assert (flat / "model" / "huggingface" / "config.json").exists()
    assert os.stat(flat / "mp_rank_00_000" / "model.pt").st_ino == os.stat(flat / "model" / "dist_ckpt" / "mp_rank_00_000" / "model.pt").st_ino
    assert migrate_layout(str(flat)) == man  # idempotent
