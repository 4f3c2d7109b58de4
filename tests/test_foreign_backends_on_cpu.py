"""Backend names of other training runtimes keep the layout they were configured with: option translation, and a 2-rank
run where ``torchtitan`` with ``tensor_parallel_size=2`` trains on the tensor-parallel engine to the single-rank result."""
import os
import socket
import warnings

import pytest
import torch
import torch.multiprocessing as mp


def test_option_names_are_translated_onto_the_two_engines():
    from verl_b200.workers.config import (AutomodelEngineConfig, FSDPEngineConfig, McoreEngineConfig, TorchtitanEngineConfig,
                                          VeOmniEngineConfig)
    from verl_b200.workers.engine.backends import translate

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        name, cfg = translate("veomni", VeOmniEngineConfig(ulysses_parallel_size=2, fsdp_size=4, enable_full_shard=True,
                                                           enable_fsdp_offload=True, seed=7, use_dynamic_bsz=True,
                                                           max_token_len_per_gpu=999))
        assert name == "native" and isinstance(cfg, FSDPEngineConfig)
        assert (cfg.ulysses_sequence_parallel_size, cfg.fsdp_size, cfg.zero_stage, cfg.optimizer_offload) == (2, 4, 3, True)
        assert (cfg.seed, cfg.use_dynamic_bsz, cfg.max_token_len_per_gpu) == (7, True, 999)
        name, cfg = translate("veomni", VeOmniEngineConfig(expert_parallel_size=4))
        assert name == "mp" and isinstance(cfg, McoreEngineConfig) and cfg.expert_model_parallel_size == 4
        name, cfg = translate("torchtitan", TorchtitanEngineConfig(tensor_parallel_size=2, pipeline_parallel_size=2, context_parallel_size=2,
                                                                  expert_tensor_parallel_size=2, activation_checkpoint="none"))
        assert name == "mp" and (cfg.tensor_model_parallel_size, cfg.pipeline_model_parallel_size, cfg.context_parallel_size,
                                 cfg.expert_tensor_parallel_size, cfg.enable_gradient_checkpointing, cfg.sequence_parallel) == (2, 2, 2, 2, False, True)
        name, cfg = translate("torchtitan", TorchtitanEngineConfig(data_parallel_shard_size=4, data_parallel_replicate_size=2,
                                                                  context_parallel_size=2, offload_policy=True))
        assert name == "native" and (cfg.fsdp_size, cfg.context_parallel_size, cfg.optimizer_offload, cfg.zero_stage) == (4, 2, True, 2)
        name, cfg = translate("automodel", AutomodelEngineConfig(tp_size=2, sequence_parallel=False, activation_checkpointing=True))
        assert name == "mp" and cfg.tensor_model_parallel_size == 2 and not cfg.sequence_parallel and cfg.enable_gradient_checkpointing
        name, cfg = translate("automodel", AutomodelEngineConfig(cp_size=2))
        assert name == "native" and cfg.context_parallel_size == 2 and not cfg.enable_gradient_checkpointing
        mc = McoreEngineConfig(tensor_model_parallel_size=2)
        assert translate("mindspeed", mc) == ("mp", mc)
        assert translate("fsdp", mc) == ("fsdp", mc)
        with pytest.raises(ValueError, match="Ulysses"):
            translate("veomni", VeOmniEngineConfig(ulysses_parallel_size=2, expert_parallel_size=2))


def test_one_warning_per_backend_names_the_engine():
    from verl_b200.workers.config import TorchtitanEngineConfig
    from verl_b200.workers.engine import backends

    backends._warned.discard("torchtitan")
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        backends.translate("torchtitan", TorchtitanEngineConfig())
        backends.translate("torchtitan", TorchtitanEngineConfig())
    msgs = [str(x.message) for x in w if "torchtitan" in str(x.message)]
    assert len(msgs) == 1 and "'native' engine" in msgs[0]


def _rank(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      VERL_ENGINE_DEVICE="cpu")
    try:
        from functools import partial

        from verl_b200.models.config import get_preset
        from verl_b200.utils.distributed import initialize_global_process_group
        from verl_b200.workers.config import TorchtitanEngineConfig, OptimizerConfig
        from verl_b200.workers.engine.base import EngineRegistry
        from verl_b200.workers.utils.losses import sft_loss

        initialize_global_process_group()
        torch.manual_seed(0)
        ids = torch.randint(3, 500, (4, 24))
        am = torch.ones_like(ids)
        am[2, 19:] = 0
        data = {"input_ids": ids, "attention_mask": am, "responses": ids[:, 8:], "response_mask": am[:, 8:]}
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            eng = EngineRegistry.new("language_model", "torchtitan", model_config=get_preset("tiny-qwen2"),
                                     engine_config=TorchtitanEngineConfig(tensor_parallel_size=2, seed=5, micro_batch_size_per_gpu=2),
                                     optimizer_config=OptimizerConfig(lr=1e-3, clip_grad=1.0))
        eng.initialize()
        lp = eng.infer_batch(dict(data))["model_output"]["log_probs"].float()
        norm = float(eng.train_batch(dict(data), partial(sft_loss, None))["metrics"]["grad_norm"])
        q.put((rank, {"cls": type(eng).__module__, "tp": eng.topo.tp, "lp": lp.tolist(), "norm": norm}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_torchtitan_with_tensor_parallel_size_two_runs_tensor_parallel(monkeypatch):
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    from functools import partial

    from verl_b200.models.config import get_preset
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.base import EngineRegistry
    from verl_b200.workers.utils.losses import sft_loss

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
    torch.manual_seed(0)
    ids = torch.randint(3, 500, (4, 24))
    am = torch.ones_like(ids)
    am[2, 19:] = 0
    data = {"input_ids": ids, "attention_mask": am, "responses": ids[:, 8:], "response_mask": am[:, 8:]}
    ref = EngineRegistry.new("language_model", "fsdp", get_preset("tiny-qwen2"), FSDPEngineConfig(seed=5, micro_batch_size_per_gpu=2),
                             OptimizerConfig(lr=1e-3, clip_grad=1.0))
    ref.initialize()
    lp = ref.infer_batch(dict(data))["model_output"]["log_probs"].float()
    norm = float(ref.train_batch(dict(data), partial(sft_loss, None))["metrics"]["grad_norm"])
    m = data["response_mask"].bool()
    for r in range(2):
        assert "error" not in res[r], res[r]["error"]
        assert res[r]["cls"].endswith("mp.engine") and res[r]["tp"] == 2
        assert (torch.tensor(res[r]["lp"])[m] - lp[m]).abs().max().item() < 1e-4 and abs(res[r]["norm"] - norm) < 1e-4 * max(1.0, norm)
