"""Shared-prompt packing: log-probs, entropies, loss and every gradient equal the per-sequence packing."""
import os
from functools import partial

import torch


def _data(n_groups=2, n=3, P=10, R=8, V=500):
    g = torch.Generator().manual_seed(0)
    rows, masks = [], []
    for gi in range(n_groups):
        plen = P - gi * 3  # different prompt lengths: left padding
        prompt = torch.randint(3, V, (plen,), generator=g)
        for j in range(n):
            rlen = R - j * 2
            resp = torch.randint(3, V, (rlen,), generator=g)
            ids = torch.cat([torch.zeros(P - plen, dtype=torch.int64), prompt, resp, torch.zeros(R - rlen, dtype=torch.int64)])
            m = torch.cat([torch.zeros(P - plen), torch.ones(plen + rlen), torch.zeros(R - rlen)]).long()
            rows.append(ids)
            masks.append(m)
    ids, am = torch.stack(rows), torch.stack(masks)
    return {"input_ids": ids, "attention_mask": am, "responses": ids[:, P:], "response_mask": am[:, P:]}


def _run(share: bool, dyn: bool):
    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    os.environ["VERL_B200_SHARE_PREFIX"] = "1" if share else "0"
    from verl_b200.models import get_preset
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.utils.losses import sft_loss

    ec = FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=3, use_dynamic_bsz=dyn, max_token_len_per_gpu=40, infer_max_token_len_per_gpu=40,
                          infer_micro_batch_size_per_gpu=3)
    eng = NativeEngineWithLMHead(get_preset("tiny-qwen2"), ec, OptimizerConfig(lr=1e-3))
    eng.initialize()
    data = _data()
    eng.optimizer_zero_grad()
    out = eng.forward_backward_batch(dict(data, calculate_entropy=True), partial(sft_loss, None), forward_only=False)
    return out["model_output"]["log_probs"].clone(), out["model_output"]["entropy"].clone(), eng.params.main_grad.clone(), eng


def test_shared_prefix_matches_plain_packing():
    for dyn in (False, True):
        lp0, en0, g0, _ = _run(False, dyn)
        lp1, en1, g1, eng = _run(True, dyn)
        assert torch.allclose(lp0, lp1, atol=1e-5) and torch.allclose(en0, en1, atol=1e-5)
        assert torch.allclose(g0, g1, atol=1e-5), (g0 - g1).abs().max()
    os.environ["VERL_B200_SHARE_PREFIX"] = "1"


def test_shared_prefix_stream_is_shorter():
    from verl_b200.workers.engine.native.engine import pack_shared_prefix_batch, prompt_group_ids

    d = _data()
    gids = prompt_group_ids(d["input_ids"], d["attention_mask"], 8)
    assert gids == [0, 0, 0, 1, 1, 1]
    batch, pos, lab, valid = pack_shared_prefix_batch(d["input_ids"], d["attention_mask"], None, 8, gids)
    assert batch.num_tokens == (10 + 8 + 6 + 4) + (7 + 8 + 6 + 4) and batch.expand_index.numel() == 3 * 10 + 3 * 7 + 2 * 18
    assert pos.numel() == lab.numel() == int(valid.sum()) and (pos[0] == 9) and (pos[8] == 9)  # shared last prompt token
