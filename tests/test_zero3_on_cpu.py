"""zero_stage=3 (working weights sharded per unit, gathered around their use, gradients reduce-scattered per unit) gives
the same update as zero_stage=2 (replicated working weights): two gloo ranks, tied and untied heads, gradient
accumulation over several micro-batches, recomputation, checkpoint round trip and the merged export."""
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


def _proc(rank, world, port, preset, tmp, q):
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
        res = {}
        finals = {}
        for stage in (2, 3):
            eng = NativeEngineWithLMHead(get_preset(preset), FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=2, zero_stage=stage),
                                         OptimizerConfig(lr=1e-2, clip_grad=0.05))
            eng.initialize()
            assert eng.zero3 == (stage == 3)
            norms = []
            for step in range(2):
                shard = {k: v.chunk(world)[rank] for k, v in _data(seed=step).items()}
                out = eng.train_batch(dict(shard), partial(sft_loss, None))   # 4 rows, 2 per micro-batch: two accumulation rounds
                norms.append(float(out["metrics"]["grad_norm"]))
            full = eng.gather_full_params()
            finals[stage] = (full.flat.float().clone(), norms)
            if stage == 3:
                res["owned_fraction"] = eng.params.store.numel() / full.flat.numel()
                res["gathers"], res["reduces"] = eng.params.gather_count, eng.params.reduce_count
                lp = eng.infer_batch({k: v.chunk(world)[rank] for k, v in _data(seed=5).items()})
                d = os.path.join(tmp, preset)
                eng.checkpoint_config = type("C", (), {"save_contents": ["model", "optimizer", "extra", "hf_model"],
                                                       "load_contents": ["model", "optimizer", "extra"]})()
                eng.save_checkpoint(d)
                eng2 = NativeEngineWithLMHead(get_preset(preset), FSDPEngineConfig(seed=99, micro_batch_size_per_gpu=2, zero_stage=3),
                                              OptimizerConfig(lr=1e-2, clip_grad=0.05))
                eng2.initialize()
                eng2.load_checkpoint(d)
                res["reload_equal"] = bool(torch.equal(eng2.gather_full_params().flat, full.flat) and torch.equal(eng2.exp_avg, eng.exp_avg)
                                           and eng2.opt_step_count == 2)
                eng_z2 = NativeEngineWithLMHead(get_preset(preset), FSDPEngineConfig(seed=99, micro_batch_size_per_gpu=2), OptimizerConfig(lr=1e-2))
                eng_z2.initialize()
                try:
                    eng_z2.load_checkpoint(d)
                    res["cross_stage_refused"] = False
                except RuntimeError as e:
                    res["cross_stage_refused"] = "zero_stage" in str(e)
        res["param_diff"] = (finals[2][0] - finals[3][0]).abs().max().item()
        res["norms"] = (finals[2][1], finals[3][1])
        q.put((rank, res))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


@pytest.mark.parametrize("preset", ["tiny-llama", "tiny-qwen2"])
def test_zero3_matches_zero2(preset, tmp_path):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_proc, args=(r, 2, port, preset, str(tmp_path), q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    for r in range(2):
        assert "error" not in res[r], res[r]["error"]
        assert res[r]["param_diff"] < 5e-5, res[r]  # one lr-sized Adam step is 1e-2: reduction order differs, values agree
        for a, b in zip(*res[r]["norms"]):
            assert abs(a - b) < 1e-5 * max(1.0, a)
        assert 0.45 < res[r]["owned_fraction"] < 0.75          # half of the weights (plus chunk padding on a tiny model)
        assert res[r]["reduces"] > 0 and res[r]["gathers"] > 0
        assert res[r]["reload_equal"] and res[r]["cross_stage_refused"]
    # the merged export of the unit-sharded checkpoint equals the gathered model
    from verl_b200.model_merger.base_model_merger import ModelMergerConfig
    from verl_b200.model_merger.fsdp_model_merger import FSDPModelMerger

    d = os.path.join(str(tmp_path), preset)
    merged = FSDPModelMerger(ModelMergerConfig(operation="merge", backend="fsdp", local_dir=d, target_dir=os.path.join(d, "out"),
                                               hf_model_config_path=os.path.join(d, "huggingface"))).merge_state_dict()
    from safetensors.torch import load_file

    exported = {}
    for f in os.listdir(os.path.join(d, "huggingface")):
        if f.endswith(".safetensors"):
            exported.update(load_file(os.path.join(d, "huggingface", f)))
    assert exported, "hf_model export missing"
    for k, v in exported.items():
        assert torch.allclose(merged[k].float(), v.float(), atol=1e-2), k


def test_optimizer_offload_matches_resident_state(tmp_path):
    """``optimizer_offload``: the chunk walk over host-resident Adam moments (three chunks here) gives the weights of the
    engine that keeps its state in place, and a checkpoint written from the offloaded state loads into a plain engine."""
    import torch
    from functools import partial

    from verl_b200.models import ModelConfig
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.utils.losses import sft_loss

    arch = ModelConfig(model_type="qwen2", vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=8, eos_token_id=2, pad_token_id=0)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(3, 128, (4, 12), generator=g)
    data = {"input_ids": ids, "attention_mask": torch.ones_like(ids), "responses": ids[:, -6:], "response_mask": torch.ones(4, 6, dtype=torch.long)}

    def make(offload, params=False):
        e = NativeEngineWithLMHead(arch, FSDPEngineConfig(seed=3, micro_batch_size_per_gpu=2, optimizer_offload=offload, param_offload=params),
                                   OptimizerConfig(lr=1e-2, clip_grad=1.0, weight_decay=0.1))
        e.initialize()
        return e

    plain, off, off_all = make(False), make(True), make(True, True)
    assert off._offloaded_states == ("exp_avg", "exp_avg_sq") and off_all._offloaded_states == ("exp_avg", "exp_avg_sq", "master")
    for e in (off, off_all):
        e.offload_chunk_elems = -(-e.master.numel() // 3)
    for _ in range(3):
        outs = [e.train_batch(dict(data), partial(sft_loss, None)) for e in (plain, off, off_all)]
        assert abs(float(outs[0]["loss"]) - float(outs[1]["loss"])) < 1e-6 and abs(float(outs[0]["loss"]) - float(outs[2]["loss"])) < 1e-6
    for e in (off, off_all):
        assert torch.allclose(plain.params.flat, e.params.flat, atol=1e-7)
        assert torch.allclose(plain.exp_avg_sq, e.exp_avg_sq, atol=1e-10) and torch.allclose(plain.master, e.master, atol=1e-7)
    off.save_checkpoint(str(tmp_path / "c"))
    fresh = make(False)
    fresh.load_checkpoint(str(tmp_path / "c"))
    assert torch.equal(fresh.exp_avg, off.exp_avg) and torch.equal(fresh.master, off.master) and fresh.opt_step_count == 3
