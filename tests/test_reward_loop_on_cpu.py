"""Reward loop: rule scoring per trajectory, DAPO over-length penalty, token bucket, reward-model routing."""
import asyncio

import numpy as np
import torch

from verl_b200.experimental.reward_loop import RewardLoopManager, RewardModelManager, RewardLoopWorker
from verl_b200.experimental.reward_loop.reward_manager import AsyncTokenBucket
from verl_b200.experimental.reward_loop.router import NaiveRouter
from verl_b200.protocol import DataProto


def _batch(n=3, P=4, R=6):
    ids = torch.arange(n * (P + R)).view(n, P + R) % 50 + 3
    am = torch.ones(n, P + R, dtype=torch.int64)
    am[0, -2:] = 0
    non = {"data_source": np.array(["custom"] * n, dtype=object),
           "reward_model": np.array([{"ground_truth": str(i)} for i in range(n)], dtype=object)}
    return DataProto.from_dict(tensors={"prompts": ids[:, :P], "responses": ids[:, P:], "input_ids": ids, "attention_mask": am}, non_tensors=non)


def test_manager_places_scores_on_last_valid_token_and_collects_extras():
    def score(data_source, solution_str, ground_truth, extra_info=None, **kw):
        return {"score": float(ground_truth) + 0.5, "n_tok": len(solution_str.split())}

    mgr = RewardLoopManager({"reward_model": {"reward_manager": "naive"}}, tokenizer=None, num_workers=2, compute_score=score)
    out = mgr.compute_rm_score(_batch())
    rs = out.batch["rm_scores"]
    assert rs[0, 3] == 0.5 and rs[0].sum() == 0.5 and rs[1, 5] == 1.5 and rs[2, 5] == 2.5
    assert list(out.non_tensor_batch["n_tok"]) == [4, 6, 6]


def test_dapo_overlong_penalty():
    cfg = {"reward_model": {"reward_manager": "dapo", "reward_kwargs": {"max_resp_len": 6, "overlong_buffer_cfg": {"enable": True, "len": 4, "penalty_factor": 1.0, "log": True}}}}
    w = RewardLoopWorker(cfg, compute_score=lambda **kw: 1.0)
    res = asyncio.run(w.compute_score_batch(_batch()))
    assert res[0]["reward_score"] == 0.5 and res[1]["reward_score"] == 0.0  # 4 resp. 6 tokens: 2 resp. 4 over the 2 free ones
    assert res[1]["reward_extra_info"]["overlong"] is True


def test_token_bucket_with_fake_clock():
    now = [0.0]
    slept = []

    async def fake_sleep(s):
        slept.append(s)
        now[0] += s

    async def go():
        b = AsyncTokenBucket(rate_limit=2.0, max_tokens=2.0, clock=lambda: now[0], sleep=fake_sleep)
        await b.acquire(2.0)   # bucket starts full
        await b.acquire(1.0)   # needs 0.5 s of refill
        await b.acquire(5.0)   # larger than the bucket: taken in pieces
        return b

    asyncio.run(go())
    assert abs(slept[0] - 0.5) < 1e-9 and abs(sum(slept) - 3.0) < 1e-9


def test_reward_model_router_batches_and_fails_over():
    from verl_b200.models import DecoderModel, FlatParams, get_preset

    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32, value_head=True)
    P.init_weights(seed=2, std=0.1)
    rm = RewardModelManager.from_models([DecoderModel(cfg, P)])

    class Broken:
        async def score(self, ids, **kw):
            raise RuntimeError("down")

    router = NaiveRouter([Broken(), rm.servers[0]])
    w = RewardLoopWorker({"reward": {"reward_model": {"enable": True}}}, reward_router=router)
    res = asyncio.run(w.compute_score_batch(_batch()))
    assert rm.servers[0].num_forwards <= 2 and router.failures[0] >= 1
    direct = rm.servers[0]._forward([_batch().batch["input_ids"][1].tolist()])[0]
    assert abs(res[1]["reward_score"] - direct) < 1e-5
