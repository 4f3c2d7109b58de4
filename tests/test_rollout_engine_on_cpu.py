"""Continuous batching + paged KV: generation must equal token-by-token greedy decoding of the full model."""
import torch

from verl_b200.models import DecoderModel, FlatParams, PackedBatch, get_preset
from verl_b200.workers.rollout.native.engine import RolloutEngine, SamplingParams


def _greedy_reference(model, prompt, n):
    ids, out, lps = list(prompt), [], []
    for _ in range(n):
        lg = model.forward_logits(PackedBatch.from_lengths(torch.tensor(ids), [len(ids)]))[-1].float()
        t = int(lg.argmax())
        lps.append(float(torch.log_softmax(lg, -1)[t]))
        out.append(t)
        ids.append(t)
    return out, lps


def test_greedy_matches_full_forward_with_more_requests_than_slots():
    torch.manual_seed(0)
    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=3, std=0.1)
    eng = RolloutEngine(cfg, P, max_num_seqs=3, max_model_len=64, block_size=8, sync_interval=3, eos_token_id=-1)
    prompts = [[5, 6, 7, 8, 9], [10, 11, 12], [20, 21, 22, 23, 24, 25, 26], [3, 4], [7, 7, 7, 7]]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=9))
    model = DecoderModel(cfg, P)
    for p, o in zip(prompts, outs):
        ref, lps = _greedy_reference(model, p, 9)
        assert o.token_ids == ref and o.stop_reason == "length"
        assert torch.allclose(torch.tensor(o.log_probs), torch.tensor(lps), atol=1e-4)
    assert not eng.running and len(eng.free_slots) == 3 and len(eng.free_blocks) == eng.num_blocks


def test_eos_stops_and_sampling_logprobs_are_consistent():
    torch.manual_seed(0)
    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=4, std=0.2)
    eng = RolloutEngine(cfg, P, max_num_seqs=4, max_model_len=48, block_size=4, sync_interval=2)
    eng.eos = -1
    first = eng.generate([[9, 9, 9]], SamplingParams(temperature=0.0, max_tokens=6))[0]
    # stop at the first position whose greedy token has not occurred before it (j = 0 if all tokens repeat)
    j = next((i for i in range(1, 6) if first.token_ids[i] not in first.token_ids[:i]), 0)
    eng.eos = first.token_ids[j]
    again = eng.generate([[9, 9, 9]], SamplingParams(temperature=0.0, max_tokens=6))[0]
    assert again.token_ids == first.token_ids[: j + 1] and again.stop_reason == "completed"
    ign = eng.generate([[9, 9, 9]], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))[0]
    assert ign.token_ids == first.token_ids
    samp = eng.generate([[4, 5, 6]] * 3, SamplingParams(temperature=1.0, max_tokens=5, ignore_eos=True))
    model = DecoderModel(cfg, P)
    for o in samp:
        ids = [4, 5, 6]
        for t, lp in zip(o.token_ids, o.log_probs):
            lg = model.forward_logits(PackedBatch.from_lengths(torch.tensor(ids), [len(ids)]))[-1].float()
            assert abs(float(torch.log_softmax(lg, -1)[t]) - lp) < 1e-4
            ids.append(t)


def test_kv_release_resume_and_abort():
    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=5, std=0.1)
    eng = RolloutEngine(cfg, P, max_num_seqs=2, max_model_len=32, block_size=4, sync_interval=2, eos_token_id=-1)
    a = eng.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=4))[0].token_ids
    eng.release_kv_cache()
    assert eng.kv is None
    eng.resume_kv_cache()
    assert eng.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=4))[0].token_ids == a
    for p in ([1, 2], [3, 4], [5, 6]):
        eng.add_request(p, SamplingParams(temperature=0.0, max_tokens=20))
    eng.step()
    aborted = eng.abort()
    done = eng.finished + aborted
    assert not eng.has_unfinished() and any(o.stop_reason == "aborted" for o in done)
    assert len(eng.free_slots) == 2 and len(eng.free_blocks) == eng.num_blocks


def test_fp8_rollout_weights_stay_close_to_bf16_and_refresh_after_updates():
    torch.manual_seed(0)
    from verl_b200.models.config import ModelConfig

    cfg = ModelConfig(model_type="qwen2", vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=32, eos_token_id=-1, pad_token_id=0)
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=3, std=0.1)
    ref = RolloutEngine(cfg, P, max_num_seqs=2, max_model_len=32, block_size=8, eos_token_id=-1)
    q8 = RolloutEngine(cfg, P, max_num_seqs=2, max_model_len=32, block_size=8, eos_token_id=-1, quantization="fp8")
    assert len(q8.model.fp8_weights) == 2 * 4
    prompts = [[5, 6, 7, 8], [9, 10, 11]]
    a = ref.generate(prompts, SamplingParams(temperature=0.0, max_tokens=4))
    b = q8.generate(prompts, SamplingParams(temperature=0.0, max_tokens=4))
    lp = max(abs(x - y) for o, p in zip(a, b) for x, y in zip(o.log_probs[:1], p.log_probs[:1]))
    assert lp < 0.6  # first-token log-prob under e4m3 weights and activations stays near the full-precision one
    old = next(iter(q8.model.fp8_weights.values()))[0].clone()
    P.flat.mul_(1.5)
    q8.clear_kv_cache()
    new = next(iter(q8.model.fp8_weights.values()))
    assert torch.equal(new[0], old) and new[1].mean() > 0  # same e4m3 codes, larger scales: the copy was rebuilt


def test_identical_prompts_are_prefilled_once_and_match_unshared_generation():
    torch.manual_seed(0)
    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=3, std=0.1)
    prompts = [[5, 6, 7, 8, 9, 10, 11, 12, 13]] * 3 + [[20, 21, 22]] * 2 + [[30, 31]]
    outs = {}
    for share in (True, False):
        eng = RolloutEngine(cfg, P, max_num_seqs=8, max_model_len=64, block_size=4, eos_token_id=-1, share_prefill=share)
        outs[share] = eng.generate(prompts, SamplingParams(temperature=1.0, max_tokens=6, seed=None))
        if share:
            assert eng.stats["prefill_tokens_shared"] == 2 * 9 + 3 and eng.stats["prefill_tokens"] == 9 * 3 + 3 * 2 + 2
        # every block came back exactly once (prompt pages shared by a group are freed by their last user)
        assert sorted(eng.free_blocks) == list(range(eng.num_blocks)) and not eng._block_users
    for a, b in zip(outs[True], outs[False]):
        assert a.token_ids == b.token_ids and max(abs(x - y) for x, y in zip(a.log_probs, b.log_probs)) < 1e-5
    assert outs[True][0].token_ids != outs[True][1].token_ids  # same prompt, different seeds: different samples


def test_stop_tokens_and_repetition_penalty():
    torch.manual_seed(0)
    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=3, std=0.1)
    prompt = [5, 6, 7, 8, 9]
    eng = RolloutEngine(cfg, P, max_num_seqs=4, max_model_len=64, block_size=4, eos_token_id=-1)
    base = eng.generate([prompt], SamplingParams(temperature=0.0, max_tokens=12))[0]
    assert base.stop_reason == "length" and len(base.token_ids) == 12
    # the 4th greedy token as a stop token: generation ends there, with the stop token as last token
    stop = base.token_ids[3]
    first = base.token_ids.index(stop)
    out = eng.generate([prompt], SamplingParams(temperature=0.0, max_tokens=12, stop_token_ids=[stop]))[0]
    assert out.token_ids == base.token_ids[: first + 1] and out.stop_reason == "completed"
    # a very large penalty under greedy decoding: no token of the prompt or of the output repeats
    pen = eng.generate([prompt, prompt], SamplingParams(temperature=0.0, max_tokens=12, repetition_penalty=1e4))
    for o in pen:
        seq = prompt + o.token_ids
        assert len(set(seq)) == len(seq), seq
    # penalty 1.0 alongside: unchanged output for that request
    again = eng.generate([prompt], SamplingParams(temperature=0.0, max_tokens=12))[0]
    assert again.token_ids == base.token_ids


def test_prometheus_export_of_engine_counters():
    from prometheus_client import generate_latest

    from verl_b200.workers.rollout.metrics import RolloutMetricsExporter

    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=3, std=0.1)
    eng = RolloutEngine(cfg, P, max_num_seqs=4, max_model_len=64, block_size=4, eos_token_id=-1)
    exp = RolloutMetricsExporter(replica="3")
    eng.generate([[5, 6, 7], [8, 9]], SamplingParams(temperature=0.0, max_tokens=5))
    exp.update(eng)
    eng.generate([[5, 6, 7]], SamplingParams(temperature=0.0, max_tokens=4))
    exp.update(eng)
    text = generate_latest(exp.registry).decode()
    assert 'verl_rollout_generated_tokens_total{replica="3"} 14.0' in text
    assert 'verl_rollout_prefill_tokens_total{replica="3"} 8.0' in text
    assert 'verl_rollout_running_requests{replica="3"} 0.0' in text and 'verl_rollout_kv_usage{replica="3"} 0.0' in text


def test_prefill_decode_disaggregation_matches_a_single_engine():
    from verl_b200.workers.rollout.pd_disaggregation import DisaggregationConfig, PrefillDecodeRollout

    torch.manual_seed(0)
    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=3, std=0.1)
    prompts = [[5, 6, 7, 8, 9, 10, 11], [20, 21, 22], [30, 31, 32, 33, 34], [5, 6, 7, 8, 9, 10, 11]]
    sp = SamplingParams(temperature=1.0, max_tokens=7)
    mk = lambda: RolloutEngine(cfg, P, max_num_seqs=4, max_model_len=64, block_size=4, eos_token_id=-1, seed=0)
    ref = mk().generate(prompts, sp)
    pd = PrefillDecodeRollout(mk(), mk(), DisaggregationConfig(enable=True, prefill_chunk=3))
    out = pd.generate(prompts, sp)
    for a, b in zip(out, ref):
        assert a.token_ids == b.token_ids and max(abs(x - y) for x, y in zip(a.log_probs, b.log_probs)) < 1e-5
    assert pd.stats["handoffs"] == 4 and pd.stats["kv_bytes_transferred"] > 0
    for eng in (pd.prefill, pd.decode):   # both stages gave every block and slot back
        assert sorted(eng.free_blocks) == list(range(eng.num_blocks)) and len(eng.free_slots) == eng.S
