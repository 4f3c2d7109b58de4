"""One generate call per sample. Parity target: ``verl/experimental/agent_loop/single_turn_agent_loop.py`` (:28-107)."""

from __future__ import annotations

import time
from typing import Any
from uuid import uuid4

from .agent_loop import AgentLoopBase, AgentLoopMetrics, AgentLoopOutput, register

__all__ = ["SingleTurnAgentLoop"]


@register("single_turn_agent")
class SingleTurnAgentLoop(AgentLoopBase):
    async def run(self, sampling_params: dict[str, Any], **kwargs) -> AgentLoopOutput:
        prompt_ids = await self.prompt_ids_from(kwargs)
        t0 = time.time()
        out = await self.server_manager.generate(request_id=uuid4().hex, prompt_ids=prompt_ids, sampling_params=dict(sampling_params))
        ids = out.token_ids[: self.response_length]
        return AgentLoopOutput(prompt_ids=prompt_ids, response_ids=ids, response_mask=[1] * len(ids),
                               response_logprobs=out.log_probs[: len(ids)] if out.log_probs else None,
                               routed_experts=out.routed_experts, num_turns=2,
                               metrics=AgentLoopMetrics(generate_sequences=time.time() - t0, num_preempted=out.num_preempted or 0),
                               extra_fields=dict(out.extra_fields or {}))
