"""NVFP4 fake quantisation and quantisation-aware training on the working weights."""
import os
from functools import partial

import torch

os.environ["VERL_ENGINE_DEVICE"] = "cpu"

GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def test_fake_quant_values_lie_on_the_scaled_e2m1_grid():
    from verl_b200.utils.qat import nvfp4_fake_quantize, nvfp4_global_scale

    g = torch.Generator().manual_seed(0)
    x = torch.randn(8, 64, generator=g) * 0.1
    gs = nvfp4_global_scale(x)
    y = nvfp4_fake_quantize(x, gs)
    assert y.shape == x.shape and torch.equal(torch.sign(y)[y != 0], torch.sign(x)[y != 0])
    yb, xb = y.view(8, 4, 16), x.view(8, 4, 16)
    scale = (xb.abs().amax(-1, keepdim=True) / (6 * gs)).clamp(max=448).to(torch.float8_e4m3fn).float() * gs
    ratio = (yb.abs() / scale)
    assert ((ratio.unsqueeze(-1) - GRID).abs().amin(-1) < 1e-5).all()          # every value is grid point x block scale
    assert (y - x).abs().max() <= 0.5 * scale.max() * 2 + 1e-6                # error bounded by the widest grid step
    assert torch.equal(nvfp4_fake_quantize(y, gs), y)                          # idempotent
    # exact ties go to the even mantissa: 0.25 -> 0, 0.75 -> 1.0, 2.5 -> 2, 5 -> 4 (block scale 1: amax = 6, gs = 1/448... use gs=1)
    t = torch.tensor([[0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] + [0.0] * 8])
    out = nvfp4_fake_quantize(t, global_scale=1.0)
    assert out[0, :8].tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0]


def test_qat_engine_keeps_working_weights_quantised_and_masters_full_precision():
    from verl_b200.models import get_preset
    from verl_b200.utils.qat import nvfp4_fake_quantize
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.utils.losses import sft_loss

    ec = FSDPEngineConfig(seed=5, micro_batch_size_per_gpu=4, qat={"enable": True})
    eng = NativeEngineWithLMHead(get_preset("tiny-llama"), ec, OptimizerConfig(lr=1e-2))
    eng.initialize()
    names = eng._qat_names
    assert any("qkv_proj" in n for n in names) and not any(("embed" in n) or ("lm_head" in n) or ("norm" in n) for n in names)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(3, 500, (4, 24), generator=g)
    am = torch.ones_like(ids)
    data = {"input_ids": ids, "attention_mask": am, "responses": ids[:, -10:], "response_mask": am[:, -10:]}
    for _ in range(2):
        out = eng.train_batch(dict(data), partial(sft_loss, None))
        assert torch.isfinite(torch.tensor(out["metrics"]["grad_norm"]))
        for n in names:
            w = eng.params.views[n]
            w2 = w.view(-1, w.shape[-1])
            blocks = w2.abs().reshape(-1, 16)
            distinct = max(len(set(b.tolist())) for b in blocks[:64])
            assert distinct <= 8, (n, distinct)                                # a block holds at most the 8 e2m1 magnitudes
    o = eng.params.offsets[names[0]]
    m = eng.master[o : o + eng.params.views[names[0]].numel()]
    assert not torch.equal(m, eng.params.views[names[0]].reshape(-1).float())  # the master copy is not quantised


def test_packed_nvfp4_export_round_trips_to_the_fake_quantised_weight():
    import torch

    from verl_b200.models import FlatParams, get_preset
    from verl_b200.utils.qat.core import QATConfig, apply_qat_to_params, nvfp4_fake_quantize, qat_target_names
    from verl_b200.utils.qat.exporter import QATWeightExporter, pack_nvfp4, unpack_nvfp4

    torch.manual_seed(0)
    w = torch.randn(8, 64) * 0.3
    w[2, 16:32] = 0.0                                           # an all-zero block
    w[5, 3] = -0.0
    fq = nvfp4_fake_quantize(w)
    packed, scale, gs = pack_nvfp4(w)
    assert packed.dtype == torch.uint8 and packed.shape == (8, 32) and scale.dtype == torch.float8_e4m3fn and scale.shape == (8, 4)
    assert torch.equal(unpack_nvfp4(packed, scale, gs, dtype=torch.float32), fq)        # same grid, same scales: bit for bit
    p2, s2, g2 = pack_nvfp4(fq)                                                          # a weight already on the grid
    assert torch.equal(unpack_nvfp4(p2, s2, g2, dtype=torch.float32), fq)
    lo, hi = packed[0, 0] & 0xF, packed[0, 0] >> 4                                       # even column low nibble, odd column high
    vals = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    sc = scale[0, 0].float() * gs[0]
    for code, col in ((lo, 0), (hi, 1)):
        v = vals[int(code) & 7] * (-1 if int(code) & 8 else 1) * sc
        assert abs(float(v) - float(fq[0, col])) < 1e-7
    # exporter over a model's parameters
    cfg = QATConfig(enable=True)
    params = FlatParams(get_preset("tiny-qwen2"), dtype=torch.float32)
    params.init_weights(seed=1)
    apply_qat_to_params(params, cfg)
    targets = qat_target_names(params, cfg)
    out = dict(QATWeightExporter(cfg).export(params))
    assert targets and all(f"{n}_packed" in out and f"{n}_scale" in out and f"{n}_global_scale" in out and n not in out for n in targets)
    assert any(k.endswith("norm.weight") for k in out) and "embed_tokens.weight" in out      # passed through
    n = targets[0]
    back = unpack_nvfp4(out[f"{n}_packed"], out[f"{n}_scale"], out[f"{n}_global_scale"], dtype=torch.float32)
    assert torch.equal(back, params.views[n].view(-1, params.views[n].shape[-1]))
    assert QATWeightExporter(cfg).quantization_config()["group_size"] == 16
