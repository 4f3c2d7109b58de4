"""Sequence-tiled dense MLP: same outputs and gradients as the untiled layer."""
import os
from functools import partial

import torch

os.environ["VERL_ENGINE_DEVICE"] = "cpu"


def _run(tile: int):
    from verl_b200.models import get_preset
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.utils.losses import sft_loss

    eng = NativeEngineWithLMHead(get_preset("tiny-llama"), FSDPEngineConfig(seed=5, micro_batch_size_per_gpu=4), OptimizerConfig(lr=1e-2))
    eng.initialize()
    eng.model.mlp_tile_tokens = tile
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(3, 500, (4, 24), generator=g)
    am = torch.ones_like(ids)
    data = {"input_ids": ids, "attention_mask": am, "responses": ids[:, -10:], "response_mask": am[:, -10:]}
    lp = eng.infer_batch(dict(data))["model_output"]["log_probs"]
    out = eng.train_batch(dict(data), partial(sft_loss, None))
    return lp, out["metrics"]["grad_norm"], eng.params.flat.clone()


def test_tiled_mlp_matches_untiled():
    lp0, n0, w0 = _run(0)
    lp1, n1, w1 = _run(32)   # 96 packed tokens -> three tiles
    assert torch.allclose(lp0, lp1, atol=1e-6)
    assert abs(n0 - n1) < 1e-5 * max(1.0, n0)
    # AdamW's first step is sign-like: a gradient that is zero up to summation order may flip, everything else agrees
    assert ((w0 - w1).abs() > 1e-5).float().mean() < 1e-3


def test_tiled_mlp_config_sets_the_tile():
    from verl_b200.models import get_preset
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead

    mc = get_preset("tiny-llama")
    import types

    holder = types.SimpleNamespace(arch=mc, tiled_mlp={"enabled": True, "num_shards": 4}, lora_rank=0, path=None, local_path=None)
    eng = NativeEngineWithLMHead(holder, FSDPEngineConfig(seed=5, max_token_len_per_gpu=2048), OptimizerConfig(lr=1e-2))
    eng.initialize()
    assert eng.model.mlp_tile_tokens == 512
