"""Sharded engine checkpoint -> merged HuggingFace directory -> reload gives the same weights."""
import os
import socket

import torch


def _proc(rank, port, tmp, q):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                          VERL_ENGINE_DEVICE="cpu")
        from verl_b200.models import get_preset
        from verl_b200.utils.distributed import initialize_global_process_group
        from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
        from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead

        initialize_global_process_group()
        eng = NativeEngineWithLMHead(get_preset("tiny-qwen2"), FSDPEngineConfig(seed=5), OptimizerConfig(lr=1e-3))
        eng.initialize()
        eng.save_checkpoint(os.path.join(tmp, "actor"), global_step=1)
        if rank == 0:
            torch.save(dict(eng.params.hf_views_dict()) if hasattr(eng.params, "hf_views_dict") else {k: v.clone() for k, v in eng.params.hf_views()},
                       os.path.join(tmp, "ref.pt"))
        q.put((rank, "ok"))
    except Exception:
        import traceback

        q.put((rank, traceback.format_exc()))


def test_merge_two_rank_flat_checkpoint(tmp_path):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_proc, args=(r, port, str(tmp_path), q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    assert res[0] == "ok" and res[1] == "ok", res
    from verl_b200.model_merger.__main__ import main
    from verl_b200.utils.model import _iter_hf_tensors

    out = tmp_path / "merged"
    main(["merge", "--backend", "fsdp", "--local_dir", str(tmp_path / "actor"), "--target_dir", str(out)])
    assert (out / "config.json").exists() and (out / "model.safetensors").exists()
    ref = torch.load(tmp_path / "ref.pt")
    merged = dict(_iter_hf_tensors(str(out)))
    for k, v in ref.items():
        if k == "lm_head.weight" and k not in merged:
            continue
        assert torch.allclose(merged[k].float(), v.float(), atol=1e-2), k
    assert "model.layers.0.self_attn.q_proj.weight" in merged and "model.layers.1.mlp.gate_proj.weight" in merged
    main(["test", "--backend", "fsdp", "--local_dir", str(tmp_path / "actor"), "--test_hf_dir", str(out)])


def test_megatron_tp_merge_rules():
    from verl_b200.model_merger.megatron_model_merger import merge_tp_tensor

    a, b = torch.ones(2, 4), torch.zeros(2, 4)
    assert merge_tp_tensor("model.layers.0.self_attn.o_proj.weight", [a, b]).shape == (2, 8)
    assert merge_tp_tensor("model.layers.0.mlp.gate_proj.weight", [a, b]).shape == (4, 4)
    assert merge_tp_tensor("model.layers.0.input_layernorm.weight", [a[0], b[0]]).equal(a[0])
