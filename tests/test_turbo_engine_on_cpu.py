"""The ``fsdp_turbo`` backend: its option tree folded into the engine's fields, refusals, and a 2-rank run that trains with
fully sharded working weights to the same result as the default configuration."""
import os

import pytest
import torch
import torch.multiprocessing as mp


def test_turbo_option_tree_is_folded_into_engine_fields():
    from verl_b200.workers.config import FSDPEngineConfig
    from verl_b200.workers.engine.native.turbo import resolve_turbo_config

    ec = FSDPEngineConfig(strategy="fsdp_turbo", offload_policy=True,
                          turbo_config={"distributed": {"fully_shard_parallel_size": 2, "ulysses_parallel_size": 2,
                                                        "fsdp_plan": {"param_dtype": "bf16", "reshard_after_forward": False}}})
    out = resolve_turbo_config(ec, world=4)
    assert out.fsdp_size == 2 and out.zero_stage == 2 and out.ulysses_sequence_parallel_size == 2   # hybrid: replicated working copy
    assert out.optimizer_offload and out.reshard_after_forward is False
    assert ec.fsdp_size == -1 and ec.zero_stage == 2 and not ec.optimizer_offload    # the caller's config is left alone
    assert resolve_turbo_config(FSDPEngineConfig(strategy="fsdp_turbo"), world=4).zero_stage == 3
    assert resolve_turbo_config(FSDPEngineConfig(strategy="fsdp_turbo"), world=1).zero_stage == 2
    assert resolve_turbo_config(FSDPEngineConfig(strategy="fsdp_turbo", forward_only=True), world=4).zero_stage == 2
    with pytest.raises(ValueError, match="strategy=megatron"):
        resolve_turbo_config(FSDPEngineConfig(strategy="fsdp_turbo", turbo_config={"distributed": {"tensor_parallel_size": 2}}), 4)
    with pytest.raises(ValueError, match="Do not enable both"):
        resolve_turbo_config(FSDPEngineConfig(strategy="fsdp_turbo", ulysses_sequence_parallel_size=2,
                                              turbo_config={"distributed": {"ulysses_parallel_size": 2}}), 4)
    with pytest.raises(ValueError, match="keeps bf16"):
        resolve_turbo_config(FSDPEngineConfig(strategy="fsdp_turbo", turbo_config={"distributed": {"fsdp_plan": {"param_dtype": "fp16"}}}), 4)


def _rank(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      VERL_ENGINE_DEVICE="cpu")
    try:
        from functools import partial

        from verl_b200.models.config import get_preset
        from verl_b200.utils.distributed import initialize_global_process_group
        from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
        from verl_b200.workers.engine.base import EngineRegistry
        from verl_b200.workers.engine.native.turbo import NativeTurboEngineWithLMHead
        from verl_b200.workers.utils.losses import sft_loss

        initialize_global_process_group()
        torch.manual_seed(0)
        ids = torch.randint(3, 500, (4, 24))
        am = torch.ones_like(ids)
        am[1, 20:] = 0
        data = {"input_ids": ids, "attention_mask": am, "responses": ids[:, 8:], "response_mask": am[:, 8:]}
        local = {k: v[rank * 2:(rank + 1) * 2] for k, v in data.items()}
        out = {}
        for name in ("fsdp", "fsdp_turbo"):
            eng = EngineRegistry.new("language_model", name, get_preset("tiny-qwen2"),
                                     FSDPEngineConfig(strategy=name, seed=5, micro_batch_size_per_gpu=2), OptimizerConfig(lr=1e-3, clip_grad=1.0))
            eng.initialize()
            m = eng.train_batch(dict(local), partial(sft_loss, None))["metrics"]
            full = eng.gather_full_params().flat.float().clone()
            out[name] = (float(m["grad_norm"]), full, int(eng.engine_config.zero_stage), type(eng).__name__)
        n = min(out["fsdp"][1].numel(), out["fsdp_turbo"][1].numel())
        q.put((rank, {"norms": (out["fsdp"][0], out["fsdp_turbo"][0]), "stages": (out["fsdp"][2], out["fsdp_turbo"][2]),
                      "cls": out["fsdp_turbo"][3], "is_turbo": out["fsdp_turbo"][3] == NativeTurboEngineWithLMHead.__name__,
                      "diff": (out["fsdp"][1][:n] - out["fsdp_turbo"][1][:n]).abs().max().item()}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_turbo_backend_trains_fully_sharded_to_the_same_weights():
    import socket

    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    for r in range(2):
        assert "error" not in res[r], res[r]["error"]
        assert res[r]["is_turbo"] and res[r]["stages"] == (2, 3), res[r]
        a, b = res[r]["norms"]
        assert abs(a - b) < 1e-5 * max(1.0, a) and res[r]["diff"] < 5e-5, res[r]
