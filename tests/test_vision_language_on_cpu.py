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


def test_cached_sampling_with_images_matches_cache_free_greedy():
    from verl_b200.models.generic import GenericRolloutEngine
    from verl_b200.workers.rollout.native.engine import SamplingParams

    arch = _arch()
    eng = _engine(arch)
    P = eng.params
    ro = GenericRolloutEngine(arch, P, max_num_seqs=4, eos_token_id=-1)
    data = _batch()
    prompts = [data["input_ids"][i, :14][data["attention_mask"][i, :14].bool()].tolist() for i in range(3)]
    mm = data["multi_modal_inputs"]
    outs = ro.generate(prompts, SamplingParams(temperature=0.0, max_tokens=4), mm_inputs=mm)
    mod = P.module.eval()
    for p, o, m in zip(prompts, outs, mm):
        seq = list(p)
        for t in range(4):
            x = torch.tensor([seq])
            with torch.no_grad():
                lg = mod(input_ids=x, attention_mask=torch.ones_like(x), use_cache=False, **(m or {})).logits[0, -1].float()
            assert int(lg.argmax()) == o.token_ids[t], (t, o.token_ids)
            assert abs(float(torch.log_softmax(lg, -1)[o.token_ids[t]]) - o.log_probs[t]) < 2e-4
            seq.append(o.token_ids[t])


def test_image_and_video_preparation():
    import io

    import numpy as np
    from PIL import Image

    from verl_b200.utils.dataset.vision_utils import process_image, process_video, smart_resize

    assert smart_resize(100, 100, 28, 56 * 56, 10**6) == (112, 112)
    h, w = smart_resize(2000, 1000, 28, 56 * 56, 200 * 200)
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 200 * 200 and abs(h / w - 2.0) < 0.35
    h, w = smart_resize(20, 30, 28, 56 * 56, 10**6)
    assert h % 28 == 0 and w % 28 == 0 and h * w >= 56 * 56
    with pytest.raises(ValueError):
        smart_resize(1, 1000)
    img = Image.fromarray((np.random.RandomState(0).rand(50, 70, 3) * 255).astype(np.uint8))
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    for src in (img, {"bytes": buf.getvalue()}, {"image": img, "max_pixels": 28 * 28 * 2}, np.asarray(img)):
        out = process_image(src, image_patch_size=14)
        assert out.mode == "RGB" and out.width % 28 == 0 and out.height % 28 == 0
    assert process_image({"image": img, "max_pixels": 28 * 28 * 2}).width * process_image({"image": img, "max_pixels": 28 * 28 * 2}).height <= 28 * 28 * 2
    frames = [np.full((40, 40, 3), i, dtype=np.uint8) for i in range(60)]       # two seconds at 30 fps
    v = process_video(frames, image_patch_size=14)
    assert v.shape == (4, 3, 28, 28) and v.dtype == torch.uint8 and int(v[0, 0, 0, 0]) == 0 and int(v[-1, 0, 0, 0]) == 59
    assert process_video({"video": frames, "nframes": 7}).shape[0] == 6          # multiple of the temporal patch


class _FakeProcessor:
    """Stands in for a vision-language processor: one placeholder token per 2x2 patch block, patches of 96 numbers."""

    def apply_chat_template(self, messages, add_generation_prompt=True, tokenize=False, **kw):
        out = []
        for m in messages:
            for part in m["content"] if isinstance(m["content"], list) else [{"type": "text", "text": m["content"]}]:
                out.append({"image": "<|img|>", "video": "<|vid|>"}.get(part["type"]) or part["text"])
        return " ".join(out)

    def __call__(self, text, images=None, videos=None, return_tensors="pt"):
        ids, pix, grids = [], [], []
        it = iter(images or [])
        for word in text[0].split():
            if word == "<|img|>":
                im = next(it)
                gh, gw = im.height // 14, im.width // 14
                ids += [VSTART] + [IMG] * ((gh // 2) * (gw // 2)) + [VEND]
                pix.append(torch.zeros(gh * gw, 96))
                grids.append([1, gh, gw])
            else:
                ids.append(3 + sum(map(ord, word)) % 400)
        enc = {"input_ids": torch.tensor([ids]), "attention_mask": torch.ones(1, len(ids), dtype=torch.int64)}
        if pix:
            enc.update(pixel_values=torch.cat(pix), image_grid_thw=torch.tensor(grids))
        return enc


def test_dataset_rows_with_images_carry_processor_outputs(tmp_path):
    import numpy as np
    import pandas as pd
    from PIL import Image

    from verl_b200.utils.dataset.rl_dataset import RLHFDataset, collate_fn

    img = Image.fromarray(np.zeros((56, 84, 3), dtype=np.uint8))
    rows = [{"prompt": [{"role": "user", "content": "look <image> and answer"}], "images": [{"image": img}], "data_source": "geo"},
            {"prompt": [{"role": "user", "content": "no picture here"}], "images": [], "data_source": "geo"}]
    f = tmp_path / "d.jsonl"
    pd.DataFrame([{**r, "images": []} for r in rows]).to_json(f, orient="records", lines=True)

    class Tok:
        pad_token_id = 0
        chat_template = None

        def __call__(self, text, add_special_tokens=False):
            return {"input_ids": [3 + sum(map(ord, w)) % 400 for w in text.split()]}

    ds = RLHFDataset(str(f), Tok(), {"max_prompt_length": 16, "filter_overlong_prompts": False}, processor=_FakeProcessor())
    ds.rows = rows                                                   # (images do not survive a json round trip)
    a, b = ds[0], ds[1]
    assert a["input_ids"].shape == (16,) and int((a["input_ids"] == IMG).sum()) == (56 // 28) * (84 // 28)
    assert a["multi_modal_inputs"]["pixel_values"].shape == (4 * 6, 96) and a["multi_modal_inputs"]["image_grid_thw"].tolist() == [[1, 4, 6]]
    assert a["multi_modal_data"]["image"][0].size == (84, 56) and "images" not in a
    assert b["multi_modal_inputs"] == {} and int((b["input_ids"] == IMG).sum()) == 0
    batch = collate_fn([a, b])
    assert batch["input_ids"].shape == (2, 16) and len(batch["multi_modal_inputs"]) == 2


def _ppo_cfg(mdir, tmp):
    return ['data.train_batch_size=4', 'data.max_prompt_length=12', 'data.max_response_length=6', 'data.synthetic.num_prompts=8',
            'data.synthetic.prompt_length=12', 'data.synthetic.vocab_high=490',
            '+data.synthetic.image.grid=[4,4]', '+data.synthetic.image.merge_size=2', '+data.synthetic.image.patch_dim=96',
            '+data.synthetic.image.image_token_id=500', '+data.synthetic.image.vision_start_token_id=498',
            '+data.synthetic.image.vision_end_token_id=499',
            f'actor_rollout_ref.model.path={mdir}', 'actor_rollout_ref.rollout.n=2', 'actor_rollout_ref.actor.ppo_mini_batch_size=4',
            'actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4', 'actor_rollout_ref.actor.use_kl_loss=true',
            'actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8', 'actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=8',
            'algorithm.adv_estimator=grpo', 'reward_model.reward_manager=token_rule', 'trainer.n_gpus_per_node=1',
            'trainer.total_epochs=1', 'trainer.total_training_steps=2', 'trainer.device=cpu', 'trainer.val_before_train=false',
            'actor_rollout_ref.rollout.max_num_seqs=8', 'trainer.resume_mode=disable', 'trainer.logger=[]',
            f'trainer.default_local_dir={tmp}/ckpt', 'trainer.save_freq=-1']


def test_grpo_end_to_end_with_images(tmp_path):
    import json

    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    arch = _arch()
    mdir = tmp_path / "tiny-qwen2_5-vl"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(arch.to_hf_dict()))
    from verl_b200.trainer.main_ppo import main

    t = main(_ppo_cfg(mdir, tmp_path))
    b = t.last_batch
    assert b.batch["advantages"].shape == (8, 6) and len(b.non_tensor_batch["multi_modal_inputs"]) == 8
    assert int((b.batch["input_ids"][:, :12] == IMG).sum()) == 8 * 4
    diff = (torch.exp(b.batch["rollout_log_probs"]) - torch.exp(b.batch["old_log_probs"])).abs()[b.batch["response_mask"].bool()].max().item()
    assert diff < 1e-3, diff     # the sampler and the training forward saw the same images


def test_supervised_fine_tuning_batches_carry_images(tmp_path):
    """SFT collate -> trainer batch -> training worker: per-row processor outputs reach the engine."""
    import json

    import numpy as np

    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from verl_b200.protocol import DataProto
    from verl_b200.utils.dataset.multiturn_sft_dataset import sft_collate
    from verl_b200.workers.config import FSDPEngineConfig, HFModelConfig, OptimizerConfig, TrainingWorkerConfig
    from verl_b200.workers.engine_workers import TrainingWorker
    from verl_b200.workers.utils.losses import sft_loss

    arch = _arch()
    mdir = tmp_path / "vl"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(arch.to_hf_dict()))
    w = TrainingWorker(TrainingWorkerConfig(model_type="language_model", model_config=HFModelConfig(path=str(mdir), load_weights=False),
                                            engine_config=FSDPEngineConfig(seed=1, micro_batch_size_per_gpu=2),
                                            optimizer_config=OptimizerConfig(lr=3e-3)))
    w.reset()
    w.set_loss_fn(partial(sft_loss, None))
    g = torch.Generator().manual_seed(0)
    items = []
    for k, (gh, gw) in enumerate(((4, 4), (2, 4), (0, 0))):
        text = torch.randint(3, 490, (10 + k,), generator=g).tolist()
        n_img = (gh // 2) * (gw // 2) if gh else 0
        ids = text[:2] + ([VSTART] + [IMG] * n_img + [VEND] if n_img else []) + text[2:]
        item = {"input_ids": torch.tensor(ids), "loss_mask": torch.tensor([0] * (len(ids) - 6) + [1] * 6)}
        if gh:
            item["multi_modal_inputs"] = _image(gh, gw, k)
        items.append(item)
    batch = sft_collate(items, pad_token_id=0)
    assert len(batch["multi_modal_inputs"]) == 3 and batch["multi_modal_inputs"][2] == {}
    non = {"multi_modal_inputs": np.array(batch.pop("multi_modal_inputs") + [None], dtype=object)[:-1]}
    proto = DataProto.from_dict(tensors=batch, non_tensors=non)
    losses = [w._train_batch(proto)["loss"] for _ in range(4)]
    assert losses[-1] < losses[0], losses
