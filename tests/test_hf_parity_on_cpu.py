"""Numerical parity of the decoder with the HuggingFace implementations of the supported model families: same random
weights (loaded through the HF-name mapping), same token ids, logits compared in fp32."""
import os

import pytest
import torch

os.environ["VERL_ENGINE_DEVICE"] = "cpu"

transformers = pytest.importorskip("transformers")

COMMON = dict(vocab_size=160, hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=False)

FAMILIES = {
    "llama": ("LlamaConfig", "LlamaForCausalLM", dict(COMMON, attention_bias=False)),
    "mistral": ("MistralConfig", "MistralForCausalLM", dict(COMMON, sliding_window=None)),
    "qwen2": ("Qwen2Config", "Qwen2ForCausalLM", dict(COMMON, use_sliding_window=False)),
    "qwen2_tied": ("Qwen2Config", "Qwen2ForCausalLM", dict(COMMON, tie_word_embeddings=True, use_sliding_window=False)),
    "qwen3": ("Qwen3Config", "Qwen3ForCausalLM", dict(COMMON, head_dim=32, use_sliding_window=False)),
    "qwen3_moe": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM", dict(COMMON, head_dim=16, num_experts=4, num_experts_per_tok=2,
                                                                moe_intermediate_size=48, norm_topk_prob=True, decoder_sparse_step=1,
                                                                mlp_only_layers=[], use_sliding_window=False)),
    "qwen2_moe": ("Qwen2MoeConfig", "Qwen2MoeForCausalLM", dict(COMMON, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=48,
                                                                shared_expert_intermediate_size=80, norm_topk_prob=False,
                                                                decoder_sparse_step=1, mlp_only_layers=[], use_sliding_window=False)),
    "mixtral": ("MixtralConfig", "MixtralForCausalLM", dict(COMMON, num_local_experts=4, num_experts_per_tok=2, sliding_window=None)),
    "phi3": ("Phi3Config", "Phi3ForCausalLM", dict(COMMON, pad_token_id=0, sliding_window=None)),
    # context extensions of the rotary embedding (original context shorter than the test sequences' positions matter for)
    "llama3_rope": ("LlamaConfig", "LlamaForCausalLM", dict(COMMON, attention_bias=False, rope_scaling=dict(
        rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=16))),
    "qwen2_yarn": ("Qwen2Config", "Qwen2ForCausalLM", dict(COMMON, use_sliding_window=False, rope_scaling=dict(
        rope_type="yarn", factor=4.0, original_max_position_embeddings=32))),
    "llama_linear": ("LlamaConfig", "LlamaForCausalLM", dict(COMMON, attention_bias=False, rope_scaling=dict(rope_type="linear", factor=2.0))),
}


def _load_into(P, sd):
    """HF in-memory state dict (fused expert tensors in recent transformers) -> flat parameters."""
    sd = dict(sd)
    missing = P.load_hf_state_dict(sd, strict=False)
    for name in missing:
        # names of the on-disk checkpoint format that the in-memory model keeps fused (experts) or renames (Mixtral router)
        if "experts" not in name and "block_sparse_moe" not in name:
            raise KeyError(name)
    for k, v in sd.items():
        if k.endswith("mlp.experts.gate_up_proj") or k.endswith("mlp.experts.down_proj") or (k.endswith("mlp.gate.weight") and "model.layers" in k):
            mine = P.views[k[len("model."):]]
            assert mine.shape == v.shape, (k, mine.shape, v.shape)
            mine.copy_(v)


@pytest.mark.parametrize("family", list(FAMILIES))
def test_logits_match_huggingface(family):
    from verl_b200.models import DecoderModel, FlatParams
    from verl_b200.models.config import ModelConfig
    from verl_b200.models.decoder import PackedBatch

    cfg_cls, model_cls, kw = FAMILIES[family]
    torch.manual_seed(0)
    hf_cfg = getattr(transformers, cfg_cls)(**kw)
    hf_cfg._attn_implementation = "eager"
    hf = getattr(transformers, model_cls)(hf_cfg).float().eval()
    for p in hf.parameters():          # biases and norms away from their trivial initial values
        if p.dim() == 1:
            p.data.add_(torch.randn_like(p) * 0.1)
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict())
    P = FlatParams(cfg, dtype=torch.float32)
    _load_into(P, hf.state_dict())
    model = DecoderModel(cfg, P)
    lens = [9, 5, 12]
    ids = [torch.randint(0, 160, (n,)) for n in lens]
    batch = PackedBatch.from_lengths(torch.cat(ids), lens, device="cpu")
    mine = model.forward_logits(batch).float()
    off = 0
    for seq, n in zip(ids, lens):
        with torch.no_grad():
            ref = hf(input_ids=seq.unsqueeze(0)).logits[0].float()
        got = mine[off : off + n]
        assert torch.allclose(got, ref, atol=2e-4, rtol=1e-3), (family, (got - ref).abs().max().item())
        off += n


def test_checkpoint_names_follow_each_family():
    from verl_b200.models import FlatParams
    from verl_b200.models.config import ModelConfig

    mix = ModelConfig.from_hf_dict(dict(COMMON, model_type="mixtral", num_local_experts=4, num_experts_per_tok=2))
    names = set(FlatParams(mix, dtype=torch.float32).hf_state_dict())
    assert {"model.layers.0.block_sparse_moe.gate.weight", "model.layers.1.block_sparse_moe.experts.3.w1.weight",
            "model.layers.1.block_sparse_moe.experts.3.w2.weight", "model.layers.1.block_sparse_moe.experts.3.w3.weight"} <= names
    assert mix.to_hf_dict()["num_local_experts"] == 4 and ModelConfig.from_hf_dict(mix.to_hf_dict()).moe_intermediate_size == 112
    phi = ModelConfig.from_hf_dict(dict(COMMON, model_type="phi3"))
    names = set(FlatParams(phi, dtype=torch.float32).hf_state_dict())
    assert "model.layers.0.self_attn.qkv_proj.weight" in names and "model.layers.0.mlp.gate_up_proj.weight" in names
    assert not any("q_proj" in n for n in names)
    q3 = ModelConfig.from_hf_dict(dict(COMMON, model_type="qwen3_moe", head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=48))
    names = set(FlatParams(q3, dtype=torch.float32).hf_state_dict())
    assert "model.layers.0.mlp.experts.2.gate_proj.weight" in names and "model.layers.0.mlp.gate.weight" in names


@pytest.mark.parametrize("family", ["qwen2", "qwen3", "qwen3_moe", "qwen2_moe", "mixtral"])
def test_gradients_match_huggingface_autograd(family):
    """The hand-scheduled backward pass against HuggingFace + autograd: gradient of the summed label log-probs with
    respect to every parameter."""
    from verl_b200.models import DecoderModel, FlatParams
    from verl_b200.models.config import ModelConfig
    from verl_b200.models.decoder import PackedBatch

    cfg_cls, model_cls, kw = FAMILIES[family]
    torch.manual_seed(1)
    hf_cfg = getattr(transformers, cfg_cls)(**kw)
    hf_cfg._attn_implementation = "eager"
    hf = getattr(transformers, model_cls)(hf_cfg).float().train()
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict())
    P = FlatParams(cfg, dtype=torch.float32, with_main_grad=True)
    _load_into(P, hf.state_dict())
    model = DecoderModel(cfg, P)
    lens = [7, 10]
    ids = [torch.randint(0, 160, (n,)) for n in lens]
    batch = PackedBatch.from_lengths(torch.cat(ids), lens, device="cpu")
    labels = torch.cat([torch.roll(s, -1) for s in ids])
    lp, _ = model.forward_logprobs(batch, labels, 1.0, need_grad=True)
    lp.sum().backward()
    total = 0.0
    for s in ids:
        logits = hf(input_ids=s.unsqueeze(0)).logits[0].float()
        ref_lp = torch.log_softmax(logits, -1).gather(-1, torch.roll(s, -1).unsqueeze(-1)).squeeze(-1)
        total = total + ref_lp.sum()
    total.backward()
    G = FlatParams(cfg, dtype=torch.float32, buffer=P.main_grad)      # the gradient buffer under the parameter names
    mine = G.hf_state_dict()
    checked = 0
    for name, p in hf.named_parameters():
        if name in mine:
            got = mine[name]
        elif name.endswith("mlp.experts.gate_up_proj") or name.endswith("mlp.experts.down_proj") or name.endswith("mlp.gate.weight"):
            got = G.views[name[len("model."):]]
        else:
            raise KeyError(name)
        scale = p.grad.abs().max().clamp(min=1e-6)
        assert (got - p.grad).abs().max() / scale < 2e-3, (family, name, float((got - p.grad).abs().max() / scale))
        checked += 1
    assert checked == len(list(hf.named_parameters()))


def test_rotary_settings_are_read_from_both_configuration_layouts():
    from verl_b200.models.config import ModelConfig

    old = dict(COMMON, model_type="llama", rope_theta=500000.0,
               rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 8192})
    new = {k: v for k, v in old.items() if k not in ("rope_theta", "rope_scaling")}
    new["rope_parameters"] = dict(old["rope_scaling"], rope_theta=500000.0)
    a, b = ModelConfig.from_hf_dict(old), ModelConfig.from_hf_dict(new)
    assert a.rope_theta == b.rope_theta == 500000.0 and a.rope_scaling == b.rope_scaling and a.rope_scaling["rope_type"] == "llama3"
    assert a.to_hf_dict()["rope_scaling"]["factor"] == 8.0 and not a.is_generic
    plain = ModelConfig.from_hf_dict(dict(COMMON, model_type="qwen2", rope_parameters={"rope_type": "default", "rope_theta": 1e6}))
    assert plain.rope_theta == 1e6 and plain.rope_scaling is None
    # rules without a hand-scheduled implementation are served by the library module instead of being ignored
    assert ModelConfig.from_hf_dict(dict(COMMON, model_type="mistral", sliding_window=16)).is_generic
    assert not ModelConfig.from_hf_dict(dict(COMMON, model_type="mistral", sliding_window=None)).is_generic
    assert not ModelConfig.from_hf_dict(dict(COMMON, model_type="qwen2", sliding_window=16, use_sliding_window=False)).is_generic
    assert ModelConfig.from_hf_dict(dict(COMMON, model_type="phi3", rope_scaling={"rope_type": "longrope", "short_factor": [1.0] * 8,
                                                                                 "long_factor": [2.0] * 8})).is_generic


def test_architecture_variants_without_a_native_implementation_use_the_library_module():
    from verl_b200.models.config import ModelConfig

    base = {k: v for k, v in COMMON.items() if k != "rope_theta"}
    generic = lambda **kw: ModelConfig.from_hf_dict(dict(base, **kw)).is_generic
    assert generic(model_type="llama", attention_bias=True)          # biases the output projection as well
    assert not generic(model_type="qwen2", attention_bias=True)
    assert generic(model_type="llama", mlp_bias=True) and generic(model_type="llama", hidden_act="gelu")
    assert generic(model_type="qwen3_moe", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, mlp_only_layers=[0])
    assert generic(model_type="qwen2_moe", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, decoder_sparse_step=2)
    assert generic(model_type="phi3", partial_rotary_factor=0.5)
    assert not generic(model_type="qwen3") and not generic(model_type="llama")
