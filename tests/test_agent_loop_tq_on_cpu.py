"""Non-blocking agent-loop manager of the replay-buffer trainers: dispatch returns at once, finished sessions land in the
replay buffer as complete groups."""
import asyncio

import torch

from tests.test_agent_loop_on_cpu import _cfg, _engines
from verl_b200 import DataProto
from verl_b200.trainer.ppo.v1.agent_loop_tq import AgentLoopManagerTQ, apply_greedy_sampling_params
from verl_b200.trainer.ppo.v1.replay_buffer import ReplayBuffer
from verl_b200.workers.rollout.llm_server import LLMServerManager


def test_greedy_params():
    sp = {"temperature": 0.7, "top_p": 0.9, "top_k": 40, "logprobs": True}
    apply_greedy_sampling_params(sp)
    assert sp == {"temperature": 0, "top_p": 1.0, "top_k": -1, "logprobs": True}


def test_dispatch_returns_at_once_and_groups_arrive_in_the_buffer():
    config = _cfg(P=8, R=6)
    rc = config.actor_rollout_ref.rollout
    rc["n"] = 2
    loop = asyncio.new_event_loop()
    mgr = loop.run_until_complete(LLMServerManager.create(rc, engines=_engines(2), model_config=None))
    rb = ReplayBuffer("sync", n=2)
    alm = AgentLoopManagerTQ.create(config, mgr, None, rb, num_workers=2, loop=loop)
    assert len(alm.workers) == 2
    ids = torch.randint(3, 500, (3, 8))
    am = torch.ones(3, 8, dtype=torch.int64)
    am[0, :2] = 0
    batch = DataProto.from_dict(tensors={"input_ids": ids, "attention_mask": am})
    assert alm.generate_sequences(batch) == 3
    assert len(alm.tasks) == 6 and rb.inflight() == 3 and not rb.ready(1)       # nothing has run yet
    alm.drain()
    assert not alm.tasks and rb.ready(3)
    meta = rb.sample(3)
    assert len(meta.keys) == 6 and len(meta.uids) == 3
    data = rb.q.get_data(meta) if hasattr(rb.q, "get_data") else None
    rb.release(meta)
    # validation: one greedy session per prompt in its own partition
    assert alm.generate_sequences(batch, validate=True) == 3 and len(alm.tasks) == 3
    alm.drain()
    assert rb.ready(3, partition_id="val", validate=True)
    loop.close()
