"""Hand-written backward of the decoder vs. autograd on a plain-PyTorch restatement; HF name round trip."""
import pytest
import torch

from verl_b200.models import DecoderModel, FlatParams, PackedBatch, get_preset
from verl_b200.models.reference import reference_logprobs, reference_values


@pytest.mark.parametrize("name", ["tiny-qwen2", "tiny-llama", "tiny-moe"])
@pytest.mark.parametrize("recompute", ["none", "full", "auto"])
def test_manual_backward_matches_autograd(name, recompute):
    torch.manual_seed(0)
    cfg = get_preset(name)
    P = FlatParams(cfg, dtype=torch.float32, with_main_grad=True)
    P.init_weights(seed=1, std=0.05)
    model = DecoderModel(cfg, P, recompute=recompute)
    model.keep_layers_fn = lambda num_tokens: 1  # "auto": the last layer keeps its activations, the others recompute
    if recompute == "full":
        from verl_b200.utils.activation_offload import ActivationOffloader

        model.offloader = ActivationOffloader("cpu")  # host device: handles pass tensors through
    lengths = [7, 12, 5]
    T = sum(lengths)
    ids = torch.randint(3, cfg.vocab_size, (T,))
    labels = torch.randint(3, cfg.vocab_size, (T,))
    w1, w2 = torch.randn(T), torch.randn(T)
    lp, ent = model.forward_logprobs(PackedBatch.from_lengths(ids, lengths), labels, 0.9)
    ((lp * w1).sum() + (ent * w2).sum()).backward()
    ref = {k: v.detach().clone().requires_grad_(True) for k, v in P.views.items()}
    lp2, ent2 = reference_logprobs(cfg, ref, ids, lengths, labels, 0.9)
    ((lp2 * w1).sum() + (ent2 * w2).sum()).backward()
    assert torch.allclose(lp, lp2, atol=1e-4) and torch.allclose(ent, ent2, atol=1e-4)
    for k, v in P.views.items():
        g = ref[k].grad if ref[k].grad is not None else torch.zeros_like(v)
        assert torch.allclose(v.main_grad, g, atol=2e-4 * max(1.0, g.abs().max().item())), k


def test_value_head_backward():
    torch.manual_seed(0)
    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32, with_main_grad=True, value_head=True)
    P.init_weights(seed=2, std=0.05)
    model = DecoderModel(cfg, P)
    lengths = [6, 9]
    ids = torch.randint(3, cfg.vocab_size, (15,))
    w = torch.randn(15)
    v = model.forward_values(PackedBatch.from_lengths(ids, lengths))
    (v * w).sum().backward()
    ref = {k: t.detach().clone().requires_grad_(True) for k, t in P.views.items()}
    v2 = reference_values(cfg, ref, ids, lengths)
    (v2 * w).sum().backward()
    assert torch.allclose(v, v2, atol=1e-4)
    assert torch.allclose(P["v_head.weight"].main_grad[0], ref["v_head.weight"].grad[0], atol=1e-4)
    assert torch.allclose(P["layers.0.mlp.down_proj.weight"].main_grad, ref["layers.0.mlp.down_proj.weight"].grad, atol=1e-4)


def test_hf_name_roundtrip_and_tied_embeddings():
    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=3)
    sd = P.hf_state_dict(clone=True)
    assert "model.layers.0.self_attn.q_proj.weight" in sd and "model.layers.1.mlp.up_proj.weight" in sd
    assert sd["model.layers.0.self_attn.k_proj.weight"].shape == (cfg.kv_size, cfg.hidden_size)
    Q = FlatParams(cfg, dtype=torch.float32)
    assert Q.load_hf_state_dict(sd) == []
    assert torch.equal(Q.flat, P.flat)
    tied = get_preset("qwen2.5-0.5b")
    tied.num_hidden_layers, tied.vocab_size = 1, 1024
    T = FlatParams(tied, dtype=torch.float32)
    assert T.lm_head_weight.data_ptr() == T["embed_tokens.weight"].data_ptr()
    assert "lm_head.weight" in dict(T.hf_views())


def test_param_counts_match_known_sizes():
    assert abs(get_preset("qwen2.5-7b").num_parameters() / 1e9 - 7.62) < 0.02
    assert abs(get_preset("qwen2.5-0.5b").num_parameters() / 1e9 - 0.494) < 0.01
    assert abs(get_preset("llama-3.1-8b").num_parameters() / 1e9 - 8.03) < 0.02
    assert abs(get_preset("qwen3-30b-a3b").num_parameters() / 1e9 - 30.5) < 0.3


def test_lm_head_on_selected_positions_matches_full_head():
    torch.manual_seed(0)
    cfg = get_preset("tiny-qwen2")
    lengths = [9, 6]
    T = sum(lengths)
    ids, labels = torch.randint(3, cfg.vocab_size, (T,)), torch.randint(3, cfg.vocab_size, (T,))
    pos = torch.tensor([2, 3, 4, 7, 11, 12])
    w = torch.randn(len(pos))
    grads = []
    for use_pos in (True, False):
        P = FlatParams(cfg, dtype=torch.float32, with_main_grad=True)
        P.init_weights(seed=1, std=0.05)
        model = DecoderModel(cfg, P, recompute="none")
        lp, ent = model.forward_logprobs(PackedBatch.from_lengths(ids, lengths), labels, 1.0, positions=pos if use_pos else None)
        if not use_pos:
            lp, ent = lp[pos], ent[pos]
        ((lp * w).sum() + 0.3 * ent.sum()).backward()
        grads.append((lp.detach().clone(), P.main_grad.clone()))
    assert torch.allclose(grads[0][0], grads[1][0], atol=1e-6) and torch.allclose(grads[0][1], grads[1][1], atol=1e-6)
