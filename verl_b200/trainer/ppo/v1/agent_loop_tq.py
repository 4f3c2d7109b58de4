"""Agent-loop worker and manager of the replay-buffer trainers: sessions are dispatched without blocking and every finished
trajectory is written into the replay buffer (the trainer consumes groups from there) instead of being returned as a batch.

Parity target: ``verl/trainer/ppo/v1/agent_loop_tq.py`` (``apply_greedy_sampling_params`` :41, ``AgentLoopWorkerTQ`` :53-227,
``AgentLoopManagerTQ`` :230-257: chunk the prompts over the workers, return at once).
"""

from __future__ import annotations

import asyncio
import uuid
from typing import Any, Optional

import torch

from .replay_buffer import ReplayBuffer
from .trainer_base import AgentLoopWorkerTQ

__all__ = ["apply_greedy_sampling_params", "AgentLoopWorkerTQ", "AgentLoopManagerTQ"]


def apply_greedy_sampling_params(params: dict[str, Any]) -> None:
    """In-place switch of a sampling-parameter dict to greedy decoding (validation passes)."""
    params["top_p"] = 1.0
    params["top_k"] = -1
    params["temperature"] = 0


class AgentLoopManagerTQ:
    """Spreads prompts over ``AgentLoopWorkerTQ`` instances that share one replay buffer. ``generate_sequences`` registers
    every prompt (one group of ``n`` sessions) in the buffer, starts the sessions on the event loop and returns; whoever owns
    the loop lets it run (``pump`` / ``drain``) and reads finished groups from the buffer."""

    def __init__(self, workers: list[AgentLoopWorkerTQ], replay_buffer: ReplayBuffer, rollout_config, loop: Optional[asyncio.AbstractEventLoop] = None,
                 version_fn=lambda: 0):
        assert workers, "at least one agent-loop worker"
        self.workers, self.rb, self.rc = list(workers), replay_buffer, rollout_config
        self.loop = loop or asyncio.new_event_loop()
        self.version_fn = version_fn
        self.tasks: set = set()
        self._next = 0

    @classmethod
    def create(cls, config, server_manager, tokenizer, replay_buffer: ReplayBuffer, num_workers: Optional[int] = None,
               loop: Optional[asyncio.AbstractEventLoop] = None, version_fn=lambda: 0) -> "AgentLoopManagerTQ":
        rc = config.actor_rollout_ref.rollout
        agent = rc.get("agent") or {}
        n = int(num_workers or agent.get("num_workers", 1) or 1)
        workers = [AgentLoopWorkerTQ(config, server_manager.client(), tokenizer, None, replay_buffer=replay_buffer, version_fn=version_fn)
                   for _ in range(n)]
        return cls(workers, replay_buffer, rc, loop, version_fn)

    def _rows(self, prompts) -> list[dict]:
        if isinstance(prompts, list):
            return prompts
        tensors = dict(prompts.batch.items()) if getattr(prompts, "batch", None) is not None else {}
        non = dict(getattr(prompts, "non_tensor_batch", {}) or {})
        n = len(prompts)
        return [{**{k: v[i] for k, v in tensors.items()}, **{k: v[i] for k, v in non.items()}} for i in range(n)]

    def generate_sequences(self, prompts, validate: bool = False) -> int:
        """Start ``n`` sessions per prompt (one for validation, greedy) without waiting for them; returns the number of
        prompts dispatched. ``prompts``: a ``DataProto`` or a list of per-prompt dicts."""
        rc = self.rc
        sp = dict(temperature=float(rc.temperature), top_p=float(rc.get("top_p", 1.0)), top_k=int(rc.get("top_k", -1)), logprobs=True)
        if validate:
            apply_greedy_sampling_params(sp)
        part = "val" if validate else "train"
        rows = self._rows(prompts)
        for p in rows:
            uid = str(p.get("uid") or uuid.uuid4().hex)
            kw = {k: v for k, v in p.items() if not isinstance(v, torch.Tensor)}
            if "raw_prompt" not in kw and "input_ids" in p:
                ids, am = p["input_ids"], p.get("attention_mask")
                kw["raw_prompt_ids"] = (ids[am.bool()] if am is not None else ids).tolist()
            sessions = 1 if validate else int(rc.n)
            self.rb.add_prompt(uid, kw, self.version_fn(), part, n=sessions)
            self.rb.mark_running(uid, part)
            worker = self.workers[self._next % len(self.workers)]     # whole groups stay on one worker
            self._next += 1
            for s in range(sessions):
                t = self.loop.create_task(worker.run_session(uid, s, str(kw.get("agent_name", worker.default_loop)), sp, kw, part))
                self.tasks.add(t)
                t.add_done_callback(self.tasks.discard)
        return len(rows)

    def pump(self, seconds: float = 0.0) -> None:
        """Let the sessions (and the in-process engines behind the servers) make progress."""
        self.loop.run_until_complete(asyncio.sleep(seconds))

    def drain(self, timeout: float = 600.0) -> None:
        """Run until every dispatched session has written its trajectory."""
        async def wait():
            if self.tasks:
                await asyncio.wait_for(asyncio.gather(*list(self.tasks), return_exceptions=True), timeout)

        self.loop.run_until_complete(wait())

    def cancel(self) -> None:
        for t in list(self.tasks):
            t.cancel()
        self.pump(0.0)
