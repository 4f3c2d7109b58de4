"""Vision-language models (tiny Qwen2.5-VL) through the generic path: per-row processor outputs travel with the batch, the
packed forward equals the library's padded forward, and the engine trains the language model and the vision tower."""
import os
from functools import partial

import pytest
import torch

transformers = pytest.importorskip("transformers")
from transformers.models.auto.configuration_auto import CONFIG_MAPPING  # noqa: E402

from verl_b200.models.config import ModelConfig  # noqa: E402

IMG, VSTART, VEND = 500, 498, 499


def _arch() -> ModelConfig:
    if "qwen2_5_vl" not in CONFIG_MAPPING:
        pytest.skip("qwen2_5_vl is not in this transformers build")
    hf = CONFIG_MAPPING["qwen2_5_vl"](
        text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}, max_position_embeddings=512),
        vision_config=dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, out_hidden_size=64, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2, fullatt_block_indexes=[1], window_size=16, in_channels=3),
        image_token_id=IMG, video_token_id=501, vision_start_token_id=VSTART, vision_end_token_id=VEND, eos_token_id=2, pad_token_id=0)
    return ModelConfig.from_hf_dict(hf.to_dict())


def _image(h_patches: int, w_patches: int, seed: int):
    """Processor output of one image: flattened patches [t*h*w, channels * temporal_patch * patch * patch] and its grid."""
    g = torch.Generator().manual_seed(seed)
    return {"pixel_values": torch.randn(h_patches * w_patches, 3 * 2 * 4 * 4, generator=g),
            "image_grid_thw": torch.tensor([[1, h_patches, w_patches]])}


def _batch(P=14, R=6, seed=0):
    """Three rows, left-padded prompts: one with a 4x4-patch image (4 placeholders), one text-only, one with a 2x4 image (2)."""
    g = torch.Generator().manual_seed(seed)
    rows, mm = [], []
    for kind in ("big", "none", "small"):
        n_img = {"big": 4, "none": 0, "small": 2}[kind]
        text = torch.randint(3, 490, (5,), generator=g).tolist()
        prompt = text[:2] + ([VSTART] + [IMG] * n_img + [VEND] if n_img else []) + text[2:]
        resp = torch.randint(3, 490, (R,), generator=g).tolist()
        rows.append((prompt, resp))
        mm.append(_image(4, 4, 1) if kind == "big" else _image(2, 4, 2) if kind == "small" else None)
    ids = torch.zeros(3, P + R, dtype=torch.int64)
    am = torch.zeros(3, P + R, dtype=torch.int64)
    for i, (p, r) in enumerate(rows):
        ids[i, P - len(p) : P] = torch.tensor(p)
        am[i, P - len(p) : P] = 1
        n = R if i != 1 else R - 2                       # one row with a short response
        ids[i, P : P + n] = torch.tensor(r[:n])
        am[i, P : P + n] = 1
    return {"input_ids": ids, "attention_mask": am, "responses": ids[:, P:], "response_mask": am[:, P:], "multi_modal_inputs": mm}


def _engine(arch, **kw):
    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead

    eng = NativeEngineWithLMHead(arch, FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=kw.pop("mbs", 2)), OptimizerConfig(lr=3e-3, clip_grad=1.0))
    eng.initialize()
    return eng


def test_log_probs_equal_the_library_forward_row_by_row():
    arch = _arch()
    assert arch.is_multimodal and arch.hidden_size == 64
    eng = _engine(arch)
    assert eng.model.multimodal and type(eng.params.module).__name__ == "Qwen2_5_VLForConditionalGeneration"
    data = _batch()
    lp = eng.infer_batch(dict(data))["model_output"]["log_probs"]          # two micro-batches: rows (0, 1) and (2)
    mod = eng.params.module.eval()
    P = 14
    for i in range(3):
        m = data["attention_mask"][i].bool()
        x = data["input_ids"][i][m][None]
        kw = {k: v for k, v in (data["multi_modal_inputs"][i] or {}).items()}
        with torch.no_grad():
            logits = mod(input_ids=x, attention_mask=torch.ones_like(x), use_cache=False, **kw).logits[0].float()
        logp = torch.log_softmax(logits, -1)
        n_p = int(data["attention_mask"][i, :P].sum())
        n_r = int(data["attention_mask"][i, P:].sum())
        want = logp[n_p - 1 : n_p - 1 + n_r].gather(-1, x[0, n_p : n_p + n_r, None]).squeeze(-1)
        assert torch.allclose(lp[i, :n_r], want, atol=2e-4), (i, (lp[i, :n_r] - want).abs().max())
        assert (lp[i, n_r:] == 0).all()
    # the images matter: other pixels, other log-probs
    other = dict(data)
    other["multi_modal_inputs"] = [_image(4, 4, 9), None, _image(2, 4, 2)]
    lp2 = eng.infer_batch(other)["model_output"]["log_probs"]
    assert not torch.allclose(lp2[0], lp[0], atol=1e-4) and torch.allclose(lp2[2], lp[2], atol=1e-6)


def test_training_updates_the_vision_tower_and_reduces_the_loss():
    from verl_b200.workers.utils.losses import sft_loss

    eng = _engine(_arch(), mbs=3)
    vis = next(k for k in eng.params.views if "visual" in k and "qkv.weight" in k)
    before = eng.params.views[vis].clone()
    losses = [float(eng.train_batch(dict(_batch()), partial(sft_loss, None))["loss"]) for _ in range(5)]
    assert losses[-1] < losses[0], losses
    assert not torch.equal(before, eng.params.views[vis])


def test_text_only_families_refuse_images():
    from tests.test_generic_families_on_cpu import _arch as text_arch

    eng = _engine(text_arch("deepseek_v3"))
    data = _batch()
    data["input_ids"] = data["input_ids"].clamp_max(400)
    with pytest.raises(AssertionError, match="vision-language"):
        eng.infer_batch(data)
