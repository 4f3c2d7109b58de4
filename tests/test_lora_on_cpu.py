"""LoRA: adapter gradients equal autograd's, the base stays frozen, the merged working weights follow the adapters."""
import os
from functools import partial

import torch


def _batch():
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(3, 500, (4, 24), generator=g)
    am = torch.ones_like(ids)
    return {"input_ids": ids, "attention_mask": am, "responses": ids[:, 8:], "response_mask": am[:, 8:]}


def test_lora_gradients_match_autograd_and_training_moves_only_adapters(tmp_path):
    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from verl_b200.models import get_preset
    from verl_b200.models.reference import reference_logprobs
    from verl_b200.workers.config import FSDPEngineConfig, HFModelConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead, pack_padded_batch
    from verl_b200.workers.utils.losses import sft_loss

    mc = HFModelConfig(path="tiny-llama", load_weights=False, lora_rank=8, lora_alpha=16)
    eng = NativeEngineWithLMHead(mc, FSDPEngineConfig(seed=3, micro_batch_size_per_gpu=4), OptimizerConfig(lr=1e-2, clip_grad=0.0))
    eng.initialize()
    lora = eng.lora
    assert lora is not None and len(lora.targets) == 4 * eng.arch.num_hidden_layers
    # make B non-zero so that both adapter gradients are non-trivial, then re-merge
    for k, v in lora.views.items():
        if k.endswith("lora_B"):
            v.normal_(0, 0.02, generator=torch.Generator().manual_seed(1))
    lora.merge()
    data = _batch()
    eng.optimizer_zero_grad()
    eng.forward_backward_batch(dict(data), partial(sft_loss, None), forward_only=False)
    # autograd reference on explicit W0 + s * B A
    A = {k: v.detach().clone().requires_grad_(True) for k, v in lora.views.items()}
    W = {}
    for n, v in eng.params.views.items():
        o = eng.params.offsets[n]
        w0 = lora.base0[o : o + v.numel()].view_as(v)
        W[n] = w0 + lora.scale * (A[f"{n}.lora_B"] @ A[f"{n}.lora_A"]) if n in lora.targets else w0.clone()
    batch, labels, resp_index, resp_valid = pack_padded_batch(data["input_ids"], data["attention_mask"], None, 16)
    lens = (batch.cu_seqlens_cpu[1:] - batch.cu_seqlens_cpu[:-1]).tolist()
    lp, _ = reference_logprobs(eng.arch, W, batch.input_ids, lens, labels, 1.0)
    loss = -(lp[resp_index][resp_valid]).sum() / resp_valid.sum()
    loss.backward()
    for k, v in lora.views.items():
        assert torch.allclose(v.main_grad, A[k].grad, atol=2e-5 * max(1.0, A[k].grad.abs().max().item())), k
    assert all(getattr(v, "main_grad", None) is None for v in eng.params.views.values())  # the base has no gradient buffers
    # one optimizer step: adapters move, the frozen copy does not, the working weights are re-merged
    before_A = lora.flat.clone()
    eng.optimizer_step()
    assert not torch.equal(lora.flat, before_A)
    n0 = lora.targets[0]
    o = eng.params.offsets[n0]
    expect = lora.base0[o : o + eng.params.views[n0].numel()].view_as(eng.params.views[n0]) + lora.scale * lora.views[f"{n0}.lora_B"] @ lora.views[f"{n0}.lora_A"]
    assert torch.allclose(eng.params.views[n0], expect, atol=1e-6)
    assert eng.master.numel() == lora.numel  # optimizer state covers the adapters only
    eng.save_checkpoint(str(tmp_path / "ckpt"), global_step=1)
    assert (tmp_path / "ckpt" / "lora_adapter" / "adapter_config.json").exists() and (tmp_path / "ckpt" / "lora_adapter" / "lora_train_meta.json").exists()
