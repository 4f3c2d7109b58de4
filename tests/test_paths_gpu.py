"""Paths whose logic is covered on CPU, run here on a GPU with bf16 weights and the native kernels underneath: the prefix
cache across requests, the prefill -> decode hand-off, the Muon optimizer and a library-module model family."""
import os
from functools import partial

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module", autouse=True)
def _gpu_only():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from verl_b200.ops import native

    assert native.load(), "native library must load on a GPU box"


def _model(vocab=2048, layers=2):
    from verl_b200.models import FlatParams, ModelConfig

    cfg = ModelConfig(model_type="qwen2", vocab_size=vocab, hidden_size=512, intermediate_size=1024, num_hidden_layers=layers,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, eos_token_id=-1, pad_token_id=0)
    P = FlatParams(cfg, dtype=torch.bfloat16, device=DEV)
    P.init_weights(seed=0, std=0.05)
    return cfg, P


def _close(a, b, tol=6e-2):
    """Same lengths; log-probs agree up to the first token where a bf16 near-tie tips the other way."""
    same = 0
    for x, y in zip(a, b):
        assert len(x.token_ids) == len(y.token_ids)
        n = next((i for i, (s, t) in enumerate(zip(x.token_ids, y.token_ids)) if s != t), len(x.token_ids))
        same += n == len(x.token_ids)
        assert max(abs(s - t) for s, t in zip(x.log_probs[: max(n, 1)], y.log_probs[: max(n, 1)])) < tol
    return same


def test_prefix_cache_on_gpu():
    from verl_b200.workers.rollout.native.engine import RolloutEngine, SamplingParams

    cfg, P = _model()
    mk = lambda cache: RolloutEngine(cfg, P, max_num_seqs=4, max_model_len=256, block_size=16, num_blocks=96, sync_interval=2,
                                     eos_token_id=-1, enable_prefix_caching=cache)
    plain, cached = mk(False), mk(True)
    g = torch.Generator().manual_seed(0)
    p1 = torch.randint(3, 2048, (70,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=12, logprobs=True)
    a1, b1 = plain.generate([p1], sp), cached.generate([p1], sp)
    assert _close(a1, b1) == 1 and cached.stats.get("prefix_cache_hit_tokens", 0) == 0
    before = cached.stats["prefill_tokens"]
    a2, b2 = plain.generate([p1], sp), cached.generate([p1], sp)       # four full pages of 16 come from the cache
    assert cached.stats["prefix_cache_hit_tokens"] == 64 and cached.stats["prefill_tokens"] - before == 6
    _close(a2, b2)
    p2 = p1 + a1[0].token_ids + torch.randint(3, 2048, (9,), generator=g).tolist()   # the next turn of the conversation
    hits = cached.stats["prefix_cache_hit_tokens"]
    _close(plain.generate([p2], sp), cached.generate([p2], sp))
    assert cached.stats["prefix_cache_hit_tokens"] - hits == (70 + 12 - 1) // 16 * 16
    torch.cuda.synchronize()


def test_prefill_decode_handoff_on_gpu():
    from verl_b200.workers.rollout.native.engine import RolloutEngine, SamplingParams
    from verl_b200.workers.rollout.pd_disaggregation import DisaggregationConfig, PrefillDecodeRollout

    cfg, P = _model()
    prompts = [list(range(5, 45)), [20, 21, 22], list(range(30, 52)), list(range(5, 45))]
    sp = SamplingParams(temperature=1.0, max_tokens=9, logprobs=True)
    mk = lambda: RolloutEngine(cfg, P, max_num_seqs=4, max_model_len=128, block_size=16, num_blocks=64, eos_token_id=-1, seed=0)
    ref = mk().generate(prompts, sp)
    pd = PrefillDecodeRollout(mk(), mk(), DisaggregationConfig(enable=True, prefill_chunk=3))
    out = pd.generate(prompts, sp)
    assert _close(out, ref) >= 3
    assert pd.stats["handoffs"] == 4 and pd.stats["kv_bytes_transferred"] > 0
    for eng in (pd.prefill, pd.decode):
        assert sorted(eng.free_blocks) == list(range(eng.num_blocks)) and len(eng.free_slots) == eng.S


def _data(b=6, L=40, R=24, V=2000, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(3, V, (b, L), generator=g)
    am = torch.ones_like(ids)
    am[1, :3] = 0
    return {k: v.to(DEV) for k, v in {"input_ids": ids, "attention_mask": am, "responses": ids[:, -R:], "response_mask": am[:, -R:]}.items()}


def test_muon_trains_on_gpu():
    from verl_b200.models import ModelConfig
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.utils.losses import sft_loss

    arch = ModelConfig(model_type="qwen2", vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=128, eos_token_id=2, pad_token_id=0)
    eng = NativeEngineWithLMHead(arch, FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=3),
                                 OptimizerConfig(lr=5e-3, clip_grad=1.0, optimizer="muon", weight_decay=0.1, muon_match_adamw_update_rms=True))
    eng.initialize()
    assert eng.muon is not None and eng.device.type == "cuda"
    losses = [float(eng.train_batch(dict(_data()), partial(sft_loss, None))["loss"]) for _ in range(6)]
    assert all(l == l for l in losses) and losses[-1] < 0.9 * losses[0], losses


def test_library_module_family_on_gpu():
    """A family without a hand-scheduled decoder (Gemma-2: soft-capped logits, sliding windows) runs as the library module
    on the flat buffers: log-probs against the library's own forward on the same weights, and optimizer steps."""
    transformers = pytest.importorskip("transformers")
    from transformers.models.auto.configuration_auto import CONFIG_MAPPING

    from verl_b200.models.config import ModelConfig
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.utils.losses import sft_loss

    if "gemma2" not in CONFIG_MAPPING:
        pytest.skip("gemma2 is not in this transformers build")
    arch = ModelConfig.from_hf_dict(CONFIG_MAPPING["gemma2"](vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                                             num_attention_heads=4, num_key_value_heads=2, head_dim=64, sliding_window=16,
                                                             eos_token_id=2, pad_token_id=0).to_dict())
    assert arch.is_generic
    eng = NativeEngineWithLMHead(arch, FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=3), OptimizerConfig(lr=1e-3, clip_grad=1.0))
    eng.initialize()
    assert type(eng.model).__name__ == "GenericCausalLM" and eng.params.flat.is_cuda
    data = _data()
    lp = eng.infer_batch(dict(data))["model_output"]["log_probs"].float()
    with torch.no_grad():
        logits = eng.params.module(input_ids=data["input_ids"], attention_mask=data["attention_mask"]).logits.float()
    ref = torch.log_softmax(logits[:, :-1], -1).gather(-1, data["input_ids"][:, 1:].unsqueeze(-1)).squeeze(-1)[:, -24:]
    m = data["response_mask"].bool()
    m[1] = False  # the left-padded row: the library's padded forward and the packed forward place its positions differently
    assert (lp[m] - ref[m]).abs().max() < 1e-1
    losses = [float(eng.train_batch(dict(data), partial(sft_loss, None))["loss"]) for _ in range(4)]
    assert all(l == l for l in losses) and losses[-1] < losses[0], losses


def test_host_offload_on_gpu():
    """Adam moments streamed through the GPU from pinned host memory (several chunks, two staging buffers, three streams)
    give the weights of the engine that keeps them resident; a forward-only engine with ``param_offload`` frees its weights
    outside ``eval_mode()`` and computes the same log-probs after they come back."""
    from verl_b200.models import ModelConfig
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.utils.losses import sft_loss

    arch = ModelConfig(model_type="qwen2", vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=128, eos_token_id=2, pad_token_id=0)

    def make(**kw):
        e = NativeEngineWithLMHead(arch, FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=3, **kw),
                                   OptimizerConfig(lr=1e-3, clip_grad=1.0, weight_decay=0.1) if not kw.get("forward_only") else None)
        e.initialize()
        return e

    plain, off = make(), make(optimizer_offload=True, param_offload=True)
    if not off._offloaded_states:
        pytest.skip("not enough free host memory to page-lock the optimizer state")
    assert off.exp_avg.device.type == "cpu" and off.exp_avg.is_pinned() and off.master.device.type == "cpu"
    off.offload_chunk_elems = -(-off.master.numel() // 5) // 8 * 8
    for _ in range(3):
        a = plain.train_batch(dict(_data()), partial(sft_loss, None))
        b = off.train_batch(dict(_data()), partial(sft_loss, None))
        assert abs(float(a["loss"]) - float(b["loss"])) < 1e-6
    off._offload_sync()
    assert torch.equal(plain.params.flat, off.params.flat)
    assert torch.equal(plain.exp_avg_sq.cpu(), off.exp_avg_sq) and torch.equal(plain.master.cpu(), off.master)

    ref = make(forward_only=True, param_offload=True)
    if ref._param_host is None:
        pytest.skip("not enough free host memory to page-lock the weights")
    ref.params.flat.copy_(plain.params.flat)
    data = _data()
    with ref.eval_mode():
        lp0 = ref.infer_batch(dict(data))["model_output"]["log_probs"].clone()
    assert ref.params.flat.untyped_storage().size() == 0
    before = torch.cuda.memory_allocated()
    with ref.eval_mode():
        assert torch.cuda.memory_allocated() > before
        lp1 = ref.infer_batch(dict(data))["model_output"]["log_probs"].clone()
    assert torch.equal(lp0, lp1) and ref.params.flat.untyped_storage().size() == 0
