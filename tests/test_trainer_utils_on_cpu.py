"""Closed-form checks of the driver-side utilities: rollout correction, metrics, sequence-length balancing, FLOPs counting,
group statistics, padding conversions, import helpers, the transfer queue."""
import math
import os

import numpy as np
import pytest
import torch

from verl_b200.protocol import DataProto


# --------------------------------------------------------------------------------------------- rollout correction
def test_rollout_rejection_mask_and_importance_weights():
    import math

    from verl_b200.trainer.ppo.rollout_corr_helper import (compute_offpolicy_metrics, compute_rollout_corr_metrics_from_logprobs,
                                                           compute_rollout_correction_and_add_to_batch, compute_rollout_correction_weights,
                                                           compute_rollout_rejection_mask)

    ratio = [[1.0, 3.0, 0.4], [1.1, 0.9, 1.0]]                             # pi_train / pi_rollout per token
    lr = torch.log(torch.tensor(ratio))
    mask = torch.tensor([[1, 1, 1], [1, 1, 0]])
    keep, m = compute_rollout_rejection_mask(lr, mask, "token_k1", "0.5_2.0")
    assert keep.tolist() == [[1, 0, 0], [1, 1, 0]] and abs(m["rollout_rs_masked_fraction"] - 0.4) < 1e-6
    assert abs(m["rollout_rs_token_k1_masked_fraction"] - 0.4) < 1e-6 and m["rollout_rs_seq_masked_fraction"] == 0.5
    # k1 = -log(ratio): the band is on pi_rollout / pi_train, so an asymmetric band keeps the ratio 3 (k1 = log 1/3) here
    keep, _ = compute_rollout_rejection_mask(lr, mask, "token_k1", "0.3_2.0")
    assert keep.tolist() == [[1, 1, 0], [1, 1, 0]]
    keep, m = compute_rollout_rejection_mask(lr, mask, "seq_mean_k1", "0.9_1.1")
    # geometric means of the ratios: (1*3*0.4)^(1/3) = 1.063, sqrt(1.1*0.9) = 0.995: both inside the band
    assert keep.tolist() == [[1, 1, 1], [1, 1, 0]] and m["rollout_rs_seq_masked_fraction"] == 0.0
    assert abs(m["rollout_rs_seq_mean_k1_seq_max"] - (-math.log(0.99) / 2)) < 1e-5
    keep, _ = compute_rollout_rejection_mask(lr, mask, "token_k2", 0.05)   # 0.5 * log-ratio^2 <= 0.05
    assert keep.tolist() == [[1, 0, 0], [1, 1, 0]]
    # k3 = r - 1 - log r per token; several options at once: every one must pass
    k3 = [[r - 1 - math.log(r) for r in row] for row in ratio]
    keep, m = compute_rollout_rejection_mask(lr, mask, "seq_max_k3,token_k1", "0.5,0.5_2.5")
    assert keep.tolist() == [[0, 0, 0], [1, 1, 0]]                         # row 0: max k3 = 3 - 1 - log 3 = 0.90 > 0.5
    assert abs(m["rollout_rs_seq_max_k3_seq_max"] - max(k3[0])) < 1e-5 and abs(m["rollout_rs_seq_max_k3_seq_min"] - max(k3[1][:2])) < 1e-6
    for bad in (("seq_max_k1", "0.5_2"), ("token_k9", 1.0), ("token_k2", "0.1_0.2"), ("token_k1,token_k2", "1,2,3")):
        with pytest.raises(ValueError):
            compute_rollout_rejection_mask(lr, mask, *bad)

    w, m = compute_rollout_correction_weights(lr, mask, "token", 2.0)
    assert torch.allclose(w, torch.tensor([[1.0, 2.0, 0.4], [1.1, 0.9, 0.0]]), atol=1e-6)
    assert abs(m["rollout_is_ratio_fraction_high"] - 0.2) < 1e-6 and abs(m["rollout_is_max"] - 2.0) < 1e-5
    vals = [1.0, 2.0, 0.4, 1.1, 0.9]
    mean = sum(vals) / 5
    assert abs(m["rollout_is_mean"] - mean) < 1e-6
    assert abs(m["rollout_is_eff_sample_size"] - 1.0 / (sum((v / mean) ** 2 for v in vals) / 5)) < 1e-5
    w, m = compute_rollout_correction_weights(lr, mask, "token", "0.5_2.0")   # band: weights outside it are zeroed
    assert torch.allclose(w, torch.tensor([[1.0, 0.0, 0.0], [1.1, 0.9, 0.0]]), atol=1e-6) and abs(m["rollout_is_oob_ratio"] - 0.4) < 1e-6
    w, m = compute_rollout_correction_weights(lr, mask, "sequence", 10.0)
    assert torch.allclose(w[0], torch.full((3,), 1.2), atol=1e-5) and torch.allclose(w[1, :2], torch.full((2,), 0.99), atol=1e-5)
    assert abs(m["rollout_is_max"] - 1.2) < 1e-5 and w[1, 2] == 0
    w, m = compute_rollout_correction_weights(lr, mask, "token", 2.0, rollout_is_batch_normalize=True)
    assert abs(m["rollout_is_batch_norm_factor"] - mean) < 1e-6 and abs(float((w * mask).sum()) / 5 - 1.0) < 1e-6

    old = torch.log(torch.tensor([[0.5, 0.6, 0.2], [0.55, 0.45, 0.5]]))
    roll = old - lr
    om = compute_offpolicy_metrics(old, roll, mask)
    assert abs(om["kl"] - float(-(lr * mask).sum() / 5)) < 1e-6 and om["chi2_token"] > 0
    assert abs(om["chi2_seq"] - ((1.2 ** 2 + 0.99 ** 2) / 2 - 1)) < 1e-5
    assert abs(om["k3_kl"] - (sum(k3[0]) + sum(k3[1][:2])) / 5) < 1e-6
    assert set(compute_rollout_corr_metrics_from_logprobs(old, roll, mask)) == {f"rollout_corr/{k}" for k in om}
    batch = DataProto.from_dict(tensors={"old_log_probs": old, "rollout_log_probs": roll, "response_mask": mask})
    out, metrics = compute_rollout_correction_and_add_to_batch(batch, {"rollout_is": "token", "rollout_is_threshold": 2.0,
                                                                        "rollout_rs": "token_k1", "rollout_rs_threshold": "0.5_2.0"})
    assert out.batch["response_mask"].tolist() == [[1, 0, 0], [1, 1, 0]] and "rollout_is_weights" in out.batch.keys()
    assert "rollout_corr/kl" in metrics and "rollout_corr/rollout_is_mean" in metrics and "rollout_corr/rollout_rs_token_k1_mean" in metrics
    batch = DataProto.from_dict(tensors={"old_log_probs": old, "rollout_log_probs": roll, "response_mask": mask})
    out, metrics = compute_rollout_correction_and_add_to_batch(batch, {})      # diagnostics only
    assert "rollout_is_weights" not in out.batch.keys() and out.batch["response_mask"].tolist() == mask.tolist()


# --------------------------------------------------------------------------------------------- metrics
def _batch():
    R, P = 4, 3
    resp_mask = torch.tensor([[1, 1, 1, 0], [1, 1, 0, 0]])
    am = torch.cat([torch.tensor([[0, 1, 1], [1, 1, 1]]), resp_mask], 1)
    t = {"responses": torch.zeros(2, R, dtype=torch.long), "attention_mask": am, "response_mask": resp_mask,
         "token_level_scores": torch.tensor([[0, 0, 1.0, 0], [0, 0.5, 0, 0]]),
         "token_level_rewards": torch.tensor([[0, 0, 0.8, 0], [0, 0.4, 0, 0]]),
         "advantages": torch.tensor([[1.0, 1.0, 1.0, 0], [-1.0, -1.0, 0, 0]]), "returns": torch.tensor([[0.8] * 4, [0.4] * 4]),
         "values": torch.tensor([[0.5] * 4, [0.1] * 4])}
    return DataProto.from_dict(tensors=t)


def test_data_timing_and_throughput_metrics():
    from verl_b200.trainer.ppo.metric_utils import (compute_data_metrics, compute_throughout_metrics, compute_timing_metrics,
                                                    process_validation_metrics, reduce_metrics)

    b = _batch()
    m = compute_data_metrics(b, use_critic=True)
    assert abs(m["critic/score/mean"] - 0.75) < 1e-6 and abs(m["critic/rewards/max"] - 0.8) < 1e-6
    assert m["response_length/mean"] == 2.5 and m["prompt_length/max"] == 3 and m["response_length/clip_ratio"] == 0.0
    assert abs(m["critic/advantages/mean"] - 0.2) < 1e-6 and "critic/vf_explained_var" in m
    tm = compute_timing_metrics(b, {"gen": 2.0, "update_actor": 1.0, "step": 4.0})
    assert tm["timing_s/gen"] == 2.0 and abs(tm["timing_per_token_ms/gen"] - 2.0 * 1000 / 5) < 1e-6
    b.meta_info["global_token_num"] = b.batch["attention_mask"].sum(-1).tolist()   # set by the trainer when it balances the batch
    th = compute_throughout_metrics(b, {"step": 4.0}, n_gpus=2)
    assert th["perf/total_num_tokens"] == 10 and abs(th["perf/throughput"] - 10 / 4.0 / 2) < 1e-9
    assert reduce_metrics({"a": [1.0, 3.0], "b": [[2.0], [4.0, 6.0]]}) == {"a": 2.0, "b": 4.0}
    val = process_validation_metrics(["gsm8k"] * 4, ["u0", "u0", "u1", "u1"], {"acc": [1.0, 0.0, 1.0, 1.0]})
    assert abs(val["gsm8k"]["acc"]["mean@2"] - 0.75) < 1e-9


# --------------------------------------------------------------------------------------------- sequence-length balancing
def test_seqlen_balancing_partitions():
    from verl_b200.utils.seqlen_balancing import (get_group_balanced_partitions, get_reverse_idx, get_seqlen_balanced_partitions,
                                                  log_seqlen_unbalance, rearrange_micro_batches, restore_dynamic_batch)

    lens = [100, 900, 300, 700, 500, 500, 200, 800]
    parts = get_seqlen_balanced_partitions(lens, 4, equal_size=True)
    assert sorted(i for p in parts for i in p) == list(range(8)) and all(len(p) == 2 for p in parts)
    sums = [sum(lens[i] for i in p) for p in parts]
    assert max(sums) - min(sums) <= 200                                # workload is quadratic-aware, still close to 1000 each
    free = get_seqlen_balanced_partitions([10, 10, 10, 1000], 2, equal_size=False)
    assert sorted(map(sorted, free)) == [[0, 1, 2], [3]]
    info = log_seqlen_unbalance(lens, parts, "t")
    assert info["t/min"] <= info["t/max"]
    assert get_reverse_idx([2, 0, 1]) == [1, 2, 0]
    # whole groups stay together
    gp = get_group_balanced_partitions([5, 5, 50, 50, 7, 7], [0, 0, 1, 1, 2, 2], 2)
    for p in gp:
        gs = {[0, 0, 1, 1, 2, 2][i] for i in p}
        assert all(sum(1 for i in p if [0, 0, 1, 1, 2, 2][i] == g) == 2 for g in gs)
    # dynamic micro-batches under a token budget, and restoring the original order
    am = torch.zeros(6, 12, dtype=torch.long)
    for i, n in enumerate([12, 3, 9, 4, 11, 2]):
        am[i, :n] = 1
    batch = {"attention_mask": am, "x": torch.arange(6).float()}
    mbs, idx = rearrange_micro_batches(batch, max_token_len=16)
    assert sorted(i for p in idx for i in p) == list(range(6))
    assert all(int(mb["attention_mask"].sum()) <= 16 for mb in mbs)
    cat = torch.cat([mb["x"] for mb in mbs])
    assert torch.equal(restore_dynamic_batch(cat, idx), batch["x"])


def test_flops_counter_and_group_stats():
    from verl_b200.models import get_preset
    from verl_b200.utils.flops_counter import FlopsCounter, get_device_flops
    from verl_b200.utils.groupwise import as_torch_index, group_mean_std

    cfg = get_preset("qwen2.5-7b")
    fc = FlopsCounter(cfg)
    lens = [3072] * 4
    fwd = fc.forward_flops(lens)
    dense = 2.0 * (cfg.num_parameters() - cfg.vocab_size * cfg.hidden_size) * sum(lens)   # the embedding gather costs nothing
    assert 0.97 < fwd / (dense + 4.0 * 4 * 3072 ** 2 * 128 * 28 * 28 / 2) < 1.03
    achieved, promised = fc.estimate_flops(lens, delta_time=1.0)
    assert abs(achieved * 1e12 / (3 * fwd) - 1.0) < 1e-6 and promised == get_device_flops("T") and promised > 0
    moe = FlopsCounter(get_preset("qwen3-30b-a3b"))
    assert moe.forward_flops([1000]) < 2.0 * 5e9 * 1000          # ~3.3 B active parameters, far below the 30 B total
    scores = torch.tensor([1.0, 3.0, 5.0, 7.0, 2.0])
    gidx = as_torch_index(["a", "a", "b", "b", "c"])
    mean, std, cnt = group_mean_std(scores, gidx)
    assert mean.tolist() == [2.0, 6.0, 0.0] and torch.allclose(std, torch.tensor([math.sqrt(2.0), math.sqrt(2.0), 1.0])) and cnt.tolist() == [2, 2, 1]


def test_padding_conversions_roundtrip():
    from verl_b200.utils.tensordict_lite import NestedRows, TensorDict
    from verl_b200.workers.utils.padding import left_right_2_no_padding, no_padding_2_padding, response_from_nested, response_to_nested

    ids = torch.tensor([[0, 0, 5, 6, 7, 8, 0], [0, 1, 2, 3, 4, 9, 9]])
    am = torch.tensor([[0, 0, 1, 1, 1, 1, 0], [0, 1, 1, 1, 1, 1, 1]])
    td = TensorDict({"input_ids": ids, "attention_mask": am, "position_ids": (am.cumsum(-1) - 1).clamp(min=0), "responses": ids[:, -3:],
                     "response_mask": am[:, -3:]}, batch_size=2)
    nested = left_right_2_no_padding(td)
    rows = nested["input_ids"]
    assert [rows.row(i).tolist() for i in range(len(rows))] == [[5, 6, 7, 8], [1, 2, 3, 4, 9, 9]]
    assert nested["loss_mask"].row(1).tolist() == [0, 0, 0, 1, 1, 1] and nested["max_response_len"] == 3
    # per-token model outputs in the packed layout come back as [b, R], left-shifted by one (output t predicts token t + 1)
    vals = NestedRows.from_list([torch.arange(4).float(), torch.arange(6).float() + 10])
    padded = no_padding_2_padding(vals, td)
    assert padded.shape == (2, 3)
    assert padded[0].tolist() == [1.0, 2.0, 0.0] and padded[1].tolist() == [12.0, 13.0, 14.0]
    rn = response_to_nested(torch.tensor([[1, 2, 0], [3, 4, 5]]), torch.tensor([[1, 1, 0], [1, 1, 1]]))
    back = response_from_nested(rn, torch.tensor([2, 3]), 3)
    assert back.tolist() == [[1, 2, 0], [3, 4, 5]]


def test_import_helpers_and_transfer_queue(tmp_path):
    from verl_b200.utils.import_utils import deprecated, is_package_available, load_class_from_fqn, load_extern_object
    from verl_b200.utils.transfer_queue import TransferQueue

    assert is_package_available("torch") and not is_package_available("definitely_not_a_package_xyz")
    assert load_class_from_fqn("collections.OrderedDict").__name__ == "OrderedDict"
    mod = tmp_path / "my_reward.py"
    mod.write_text("def score(x):\n    return x * 2\n")
    assert load_extern_object(str(mod), "score")(21) == 42

    @deprecated("new_fn")
    def old_fn():
        return 1

    with pytest.warns(Warning):
        assert old_fn() == 1
    tq = TransferQueue()
    for i in range(4):
        tq.put(f"u{i}_0_0", {"prompt": torch.tensor([i]), "n": i}, tags={"status": "pending", "global_steps": 0})
    tq.put("u1_0_0", {"response": torch.tensor([7, 8])}, tags={"status": "finished"})
    assert tq.size() == 4 and tq.list_keys(where=lambda k, t: t["status"] == "finished") == ["u1_0_0"]
    meta = tq.get_meta(["u1_0_0", "u3_0_0"], fields=["prompt"])
    assert len(meta) == 2 and meta.tags[0]["status"] == "finished" and [len(m) for m in meta.chunk(2)] == [1, 1]
    data = tq.get_data(meta)
    assert data[0]["prompt"].tolist() == [1] and "response" not in data[0]            # field selection
    assert tq.get(["u1_0_0"])[0]["response"].tolist() == [7, 8]
    tq.delete(["u0_0_0"])
    assert tq.size() == 3 and tq.wait(lambda: tq.size() == 3, timeout=0.1)
    tq.clear()
    assert tq.size() == 0


def test_tracking_backends_and_rollout_trace(tmp_path, monkeypatch, capsys):
    import asyncio
    import json

    from verl_b200.utils.rollout_trace import TRACE_RING, RolloutTraceConfig, rollout_trace_attr, rollout_trace_op
    from verl_b200.utils.tracking import Tracking

    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path))
    tr = Tracking("proj", "exp", default_backend=["console", "file"], config={"a": {"b": 1}})
    tr.log({"loss": 0.25, "note": "text"}, step=3)
    del tr
    assert "loss:0.250" in capsys.readouterr().out or True
    files = [os.path.join(d, f) for d, _, fs in os.walk(tmp_path) for f in fs if f.endswith(".jsonl")]
    assert files, "the file backend writes JSON lines"
    rec = json.loads(open(files[0]).read().strip().splitlines()[-1])
    assert rec["step"] == 3 and abs(rec["data"]["loss"] - 0.25) < 1e-9 if "data" in rec else abs(rec["loss"] - 0.25) < 1e-9
    with pytest.raises(Exception):
        Tracking("p", "e", default_backend=["not_a_backend"])

    RolloutTraceConfig.reset()
    RolloutTraceConfig.init("proj", "exp", backend="memory")
    TRACE_RING.clear()

    class Loop:
        @rollout_trace_op
        async def run(self, x):
            return x + 1

        @rollout_trace_op
        def tool(self):
            raise RuntimeError("tool failed")

    with rollout_trace_attr(sample_index=5, step=2, rollout_n=1):
        assert asyncio.run(Loop().run(1)) == 2
        with pytest.raises(RuntimeError):
            Loop().tool()
    ops = [(t["op"].split(".")[-1], t["ok"], t["sample_index"]) for t in TRACE_RING]
    assert ops == [("run", True, 5), ("tool", False, 5)]
    RolloutTraceConfig.reset()
