"""Cache-free rollouts: greedy output equals the paged engine's greedy output; EOS masking; top-k/top-p filter."""
import torch

from verl_b200.models import DecoderModel, FlatParams, get_preset
from verl_b200.protocol import DataProto
from verl_b200.workers.rollout.base import get_rollout_class
from verl_b200.workers.rollout.naive.naive_rollout import filter_logits


def _build_model():
    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=3, std=0.1)
    return cfg, DecoderModel(cfg, P)


def _prompts(cfg, b=3, P=6):
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(3, cfg.vocab_size, (b, P), generator=g)
    am = torch.ones(b, P, dtype=torch.int64)
    am[0, :2] = 0  # left padding
    ids[0, :2] = 0
    pos = (am.cumsum(-1) - 1).clamp_min(0)
    return DataProto.from_dict({"input_ids": ids, "attention_mask": am, "position_ids": pos})


def test_filter_logits():
    l = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    assert torch.isinf(filter_logits(l, top_k=2)[0, :2]).all() and torch.isfinite(filter_logits(l, top_k=2)[0, 2:]).all()
    f = filter_logits(l, top_p=0.7)  # p = [.03,.09,.24,.64]: 4.0 alone is < .7 so 3.0 is kept too
    assert torch.isfinite(f[0, 2:]).all() and torch.isinf(f[0, :2]).all()


def test_hf_and_naive_rollout_greedy_agree_and_mask_after_eos():
    cfg, model = _build_model()
    prompts = _prompts(cfg)
    conf = {"response_length": 5, "temperature": 1.0, "do_sample": False, "top_k": 0, "top_p": 1.0}
    naive = get_rollout_class("naive", "sync")(model, conf, cfg)
    hf = get_rollout_class("hf", "sync")(model, conf, cfg)
    a = naive.generate_sequences(prompts)
    prompts.meta_info["eos_token_id"] = int(a.batch["responses"][1, 1])  # force an early stop on row 1
    b = hf.generate_sequences(prompts)
    assert torch.equal(a.batch["responses"][0], b.batch["responses"][0])
    r1 = b.batch["response_mask"][1]
    first = (a.batch["responses"][1] == prompts.meta_info["eos_token_id"]).nonzero()[0, 0].item()
    assert r1[: first + 1].all() and not r1[first + 1 :].any()
    assert b.batch["input_ids"].shape == (3, 11)
