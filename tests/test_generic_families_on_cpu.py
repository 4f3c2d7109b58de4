"""Architectures without a hand-scheduled decoder (DeepSeek-V3 latent attention + grouped routing, GPT-OSS sinks + sliding
windows, Gemma-2 soft-capped logits) run as library modules behind the engine's flat-buffer memory plan."""
import json
import os
from functools import partial

import pytest
import torch

transformers = pytest.importorskip("transformers")
from transformers.models.auto.configuration_auto import CONFIG_MAPPING  # noqa: E402

from verl_b200.models.config import ModelConfig  # noqa: E402
from verl_b200.models.decoder import PackedBatch  # noqa: E402
from verl_b200.models.generic import GenericCausalLM, GenericRolloutEngine, ModuleFlatParams  # noqa: E402

TINY = {
    "deepseek_v3": dict(vocab_size=512, hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=3,
                        num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1, n_routed_experts=8, kv_lora_rank=32,
                        q_lora_rank=48, qk_rope_head_dim=16, v_head_dim=32, qk_nope_head_dim=32, n_group=2, topk_group=1,
                        num_experts_per_tok=2, first_k_dense_replace=1, eos_token_id=2, pad_token_id=0),
    "gpt_oss": dict(vocab_size=512, hidden_size=128, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=32, num_local_experts=4, num_experts_per_tok=2, sliding_window=4,
                    eos_token_id=2, pad_token_id=0),
    "gemma2": dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=32, sliding_window=4, eos_token_id=2, pad_token_id=0),
}


def _arch(family: str) -> ModelConfig:
    if family not in CONFIG_MAPPING:
        pytest.skip(f"{family} is not in this transformers build")
    return ModelConfig.from_hf_dict(CONFIG_MAPPING[family](**TINY[family]).to_dict())


def _packed(lens, V=500, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(3, V, (sum(lens),), generator=g)
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    return PackedBatch(input_ids=ids, positions=pos, cu_seqlens=cu, max_seqlen=max(lens), cu_seqlens_cpu=cu)


@pytest.mark.parametrize("family", ["deepseek_v3", "gpt_oss", "gemma2"])
def test_packed_forward_and_flat_gradients_match_the_library(family):
    arch = _arch(family)
    assert arch.is_generic and arch.to_hf_dict()["model_type"] == family
    P = ModuleFlatParams(arch, dtype=torch.float32, seed=5)
    m = GenericCausalLM(arch, P, recompute="full")
    lens = [5, 9, 3]
    batch = _packed(lens)
    labels = torch.roll(batch.input_ids, -1)
    P.attach_main_grad()
    lp, ent = m.forward_logprobs(batch, labels, 0.7, need_grad=True)
    (lp.sum() + 0.3 * ent.sum()).backward()
    assert all(p.grad is None for p in P.module.parameters())            # folded into the flat fp32 buffer and dropped
    # every parameter is a view of the flat buffer
    lo, hi = P.flat.data_ptr(), P.flat.data_ptr() + P.flat.numel() * P.flat.element_size()
    assert all(lo <= p.data_ptr() < hi for p in P.module.parameters())

    # oracle: an independent copy of the module, one padded row per sequence, plain autograd
    from verl_b200.models.generic import build_hf_module

    ref = build_hf_module(arch, torch.float32, seed=5)
    ref.load_state_dict({k: v.clone() for k, v in P.hf_state_dict().items()}, strict=False)
    ref.eval()
    total, off, lps = 0.0, 0, []
    for n in lens:
        x = batch.input_ids[off : off + n][None]
        logits = ref(input_ids=x, use_cache=False).logits[0].float() / 0.7
        logp = torch.log_softmax(logits, -1)
        l_ref = logp.gather(-1, labels[off : off + n, None]).squeeze(-1)
        e_ref = -(logp.exp() * logp).sum(-1)
        total = total + l_ref.sum() + 0.3 * e_ref.sum()
        lps.append(l_ref.detach())
        off += n
    total.backward()
    assert torch.allclose(lp.detach(), torch.cat(lps), atol=2e-4), (lp.detach() - torch.cat(lps)).abs().max()
    worst = 0.0
    for name, p in ref.named_parameters():
        g = P._grad_views[name]
        rg = p.grad if p.grad is not None else torch.zeros_like(p)
        worst = max(worst, float((g - rg).abs().max() / (rg.abs().max() + 1e-6)))
    assert worst < 2e-3, worst


def test_selected_positions_and_no_grad_path():
    arch = _arch("deepseek_v3")
    P = ModuleFlatParams(arch, dtype=torch.float32, seed=1)
    m = GenericCausalLM(arch, P)
    batch = _packed([6, 4])
    labels = torch.roll(batch.input_ids, -1)
    full, _ = m.forward_logprobs(batch, labels, 1.0, need_grad=False)
    sel = torch.tensor([1, 4, 8])
    part, ent = m.forward_logprobs(batch, labels, 1.0, need_grad=False, positions=sel)
    assert not part.requires_grad and torch.allclose(part, full[sel], atol=1e-5) and ent.shape == (3,)
    other = torch.tensor([7, 8, 9])
    alt, _ = m.forward_logprobs(batch, labels, 1.0, need_grad=False, positions=sel, position_labels=other)
    logits = m.forward_logits(batch)
    assert torch.allclose(alt, torch.log_softmax(logits[sel], -1).gather(-1, other[:, None]).squeeze(-1), atol=1e-5)


def test_cached_sampling_matches_cache_free_greedy_and_reports_logprobs():
    from verl_b200.workers.rollout.naive.naive_rollout import last_token_logits
    from verl_b200.workers.rollout.native.engine import SamplingParams

    arch = _arch("deepseek_v3")
    P = ModuleFlatParams(arch, dtype=torch.float32, seed=2)
    m = GenericCausalLM(arch, P)
    eng = GenericRolloutEngine(arch, P, max_num_seqs=2, eos_token_id=-1)
    prompts = [[5, 6, 7], [8, 9, 10, 11, 12], [3, 4]]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5))
    for p, o in zip(prompts, outs):
        seq = list(p)
        for t in range(5):
            x = torch.tensor([seq])
            lg = last_token_logits(m, x, torch.ones_like(x))
            assert int(lg.argmax()) == o.token_ids[t]
            assert abs(float(torch.log_softmax(lg, -1)[0, o.token_ids[t]]) - o.log_probs[t]) < 1e-4
            seq.append(o.token_ids[t])
        assert o.stop_reason == "length" and o.prompt_ids == p
    # sampling: seeded requests repeat; a stop token ends a row early
    sp = SamplingParams(temperature=1.0, top_k=20, max_tokens=6, seed=11)
    a, b = eng.generate(prompts[:2], sp), eng.generate(prompts[:2], sp)
    assert [o.token_ids for o in a] == [o.token_ids for o in b]
    stop = a[0].token_ids[2]
    c = eng.generate(prompts[:1], SamplingParams(temperature=1.0, top_k=20, max_tokens=6, seed=11, stop_token_ids=(stop,)))
    assert c[0].token_ids[-1] == stop and len(c[0].token_ids) <= 3 and c[0].stop_reason == "completed"


def _train_data(b=6, L=20, R=12, V=500, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(3, V, (b, L), generator=g)
    am = torch.ones_like(ids)
    am[1, :3] = 0
    am[2, -4:] = 0
    return {"input_ids": ids, "attention_mask": am, "responses": ids[:, -R:], "response_mask": am[:, -R:]}


def test_engine_trains_a_generic_family_and_round_trips_checkpoints(tmp_path):
    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead, NativeEngineWithValueHead
    from verl_b200.workers.utils.losses import sft_loss

    arch = _arch("deepseek_v3")
    mk = lambda: NativeEngineWithLMHead(arch, FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=3), OptimizerConfig(lr=3e-3, clip_grad=1.0))
    eng = mk()
    eng.initialize()
    assert type(eng.model).__name__ == "GenericCausalLM" and not eng._share_prefix
    losses = [float(eng.train_batch(dict(_train_data()), partial(sft_loss, None))["loss"]) for _ in range(4)]
    assert losses[-1] < losses[0], losses
    eng.save_checkpoint(str(tmp_path))
    eng2 = mk()
    eng2.initialize()
    eng2.load_checkpoint(str(tmp_path))
    assert torch.equal(eng2.params.flat, eng.params.flat) and torch.equal(eng2.exp_avg, eng.exp_avg)
    out1 = eng.infer_batch(dict(_train_data(seed=3)))
    out2 = eng2.infer_batch(dict(_train_data(seed=3)))
    assert torch.equal(out1["model_output"]["log_probs"], out2["model_output"]["log_probs"])
    # the per-tensor weight stream carries the library's checkpoint names
    names = [n for n, _ in eng.get_per_tensor_param()[0]] if isinstance(eng.get_per_tensor_param(), tuple) else \
        [n for n, _ in eng.get_per_tensor_param()]
    assert any(n.endswith("self_attn.kv_a_proj_with_mqa.weight") for n in names)

    critic = NativeEngineWithValueHead(arch, FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=3), OptimizerConfig(lr=1e-3))
    critic.initialize()
    vals = critic.infer_batch(dict(_train_data()))["model_output"]["values"]
    assert vals.shape == (6, 12) and torch.isfinite(vals).all()


def test_native_decoder_refuses_generic_architectures():
    from verl_b200.models.decoder import DecoderModel

    arch = _arch("gpt_oss")
    with pytest.raises(AssertionError, match="hand-scheduled"):
        DecoderModel(arch, None)


def test_grpo_end_to_end_on_a_generic_family(tmp_path):
    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    arch = _arch("deepseek_v3")
    mdir = tmp_path / "tiny-deepseek-v3"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(arch.to_hf_dict()))
    from verl_b200.trainer.main_ppo import main

    t = main(['data.train_batch_size=4', 'data.max_prompt_length=8', 'data.max_response_length=6', 'data.synthetic.num_prompts=8',
              'data.synthetic.prompt_length=8', 'data.synthetic.vocab_high=512', f'actor_rollout_ref.model.path={mdir}',
              'actor_rollout_ref.rollout.n=2', 'actor_rollout_ref.actor.ppo_mini_batch_size=4',
              'actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4', 'actor_rollout_ref.actor.use_kl_loss=true',
              'actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8', 'actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=8',
              'algorithm.adv_estimator=grpo', 'reward_model.reward_manager=token_rule', 'trainer.n_gpus_per_node=1',
              'trainer.total_epochs=1', 'trainer.total_training_steps=2', 'trainer.device=cpu', 'trainer.val_before_train=false',
              'actor_rollout_ref.rollout.max_num_seqs=8', 'trainer.resume_mode=disable', 'trainer.logger=[]',
              f'trainer.default_local_dir={tmp_path}/ckpt', 'trainer.save_freq=-1'])
    b = t.last_batch.batch
    assert b["advantages"].shape == (8, 6)
    diff = (torch.exp(b["rollout_log_probs"]) - torch.exp(b["old_log_probs"])).abs()[b["response_mask"].bool()].max().item()
    assert diff < 1e-3, diff   # cached sampling and the packed training forward agree on token probabilities


def _dp_proc(rank, world, port, hf_dict, q):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                          VERL_ENGINE_DEVICE="cpu")
        from verl_b200.utils.distributed import initialize_global_process_group
        from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
        from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
        from verl_b200.workers.utils.losses import sft_loss

        initialize_global_process_group()
        eng = NativeEngineWithLMHead(ModelConfig.from_hf_dict(hf_dict), FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=3),
                                     OptimizerConfig(lr=3e-3, clip_grad=0.5))
        eng.initialize()
        shard = {k: v.chunk(world)[rank] for k, v in _train_data().items()}
        out = eng.train_batch(dict(shard), partial(sft_loss, None))
        q.put((rank, {"grad_norm": float(out["metrics"]["grad_norm"]), "flat": eng.params.flat.numpy(), "master": eng.master.numel()}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_sharded_optimizer_over_two_ranks_matches_one_rank():
    import socket

    import torch.multiprocessing as mp

    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.utils.losses import sft_loss

    arch = _arch("deepseek_v3")
    ref = NativeEngineWithLMHead(arch, FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=3), OptimizerConfig(lr=3e-3, clip_grad=0.5))
    ref.initialize()
    ref_norm = float(ref.train_batch(dict(_train_data()), partial(sft_loss, None))["metrics"]["grad_norm"])
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_dp_proc, args=(r, 2, port, arch.to_hf_dict(), q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    for r in range(2):
        assert "error" not in res[r], res[r]["error"]
        assert 0 <= res[r]["master"] * 2 - ref.params.numel < 1024              # half of the optimizer state per rank (+ padding)
        assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm)
        n = ref.params.numel
        assert torch.allclose(torch.from_numpy(res[r]["flat"])[:n], ref.params.flat, atol=2e-5)


def test_flops_estimates_follow_the_library_configuration():
    from verl_b200.utils.flops_counter import FlopsCounter, _causal_pairs

    v3 = dict(model_type="deepseek_v3", vocab_size=129280, hidden_size=7168, intermediate_size=18432, moe_intermediate_size=2048,
              num_hidden_layers=61, num_attention_heads=128, num_key_value_heads=128, n_shared_experts=1, n_routed_experts=256,
              kv_lora_rank=512, q_lora_rank=1536, qk_rope_head_dim=64, v_head_dim=128, qk_nope_head_dim=128,
              num_experts_per_tok=8, first_k_dense_replace=3)
    fc = FlopsCounter(ModelConfig.from_hf_dict(v3))
    active = fc._dense_per_token()
    assert 35e9 < active < 39e9, active            # ~37 B activated parameters per token
    # attention: 61 global layers, 128 heads, score width 192 and value width 128
    assert fc._attention_forward_flops([1000]) == 2.0 * 61 * 128 * (192 + 128) * _causal_pairs(1000)

    oss = dict(model_type="gpt_oss", vocab_size=201088, hidden_size=2880, intermediate_size=2880, num_hidden_layers=24,
               num_attention_heads=64, num_key_value_heads=8, head_dim=64, num_local_experts=32, num_experts_per_tok=4,
               sliding_window=128, layer_types=["sliding_attention", "full_attention"] * 12)
    fo = FlopsCounter(ModelConfig.from_hf_dict(oss))
    assert 2.5e9 < fo._dense_per_token() < 4.0e9   # ~3.6 B active of 21 B
    long, short = fo._attention_forward_flops([4096]), fo._attention_forward_flops([128])
    full_only = 2.0 * 24 * 64 * 128 * _causal_pairs(4096)
    assert 0.5 * full_only < long < 0.55 * full_only     # half of the layers see at most 128 keys
    assert short == 2.0 * 24 * 64 * 128 * _causal_pairs(128)
    assert _causal_pairs(10, 4) == 10 + 9 + 9 + 6      # 1+2+3+4 then 4 per query


def test_sharded_checkpoint_of_a_generic_family_merges_to_library_names(tmp_path):
    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from verl_b200.models import FlatParams, make_flat_params
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead

    arch = _arch("deepseek_v3")
    with pytest.raises(AssertionError, match="make_flat_params"):
        FlatParams(arch)
    eng = NativeEngineWithLMHead(arch, FSDPEngineConfig(seed=3), OptimizerConfig(lr=1e-3))
    eng.initialize()
    ck = tmp_path / "ckpt"
    eng.save_checkpoint(str(ck))
    hf_dir = tmp_path / "hf"
    hf_dir.mkdir()
    (hf_dir / "config.json").write_text(json.dumps(arch.to_hf_dict()))
    from verl_b200.model_merger.base_model_merger import ModelMergerConfig
    from verl_b200.model_merger.fsdp_model_merger import FSDPModelMerger

    merger = FSDPModelMerger(ModelMergerConfig(operation="merge", backend="fsdp", local_dir=str(ck), target_dir=str(tmp_path / "out"),
                                               hf_model_config_path=str(hf_dir)))
    sd = merger.merge_state_dict()
    want = eng.params.hf_state_dict()
    assert set(sd) == set(want)
    assert all(torch.allclose(sd[k].float(), want[k].float(), atol=1e-2) for k in want)       # bf16 copy of the fp32 weights
    # storage over a given buffer keeps the buffer's content
    P2 = make_flat_params(arch, dtype=torch.float32, buffer=eng.params.flat.clone())
    assert torch.equal(P2.flat, eng.params.flat)
