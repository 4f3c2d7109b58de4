"""Multi-turn tool-using agent loop as a small state machine.

PENDING -> GENERATING -> PROCESSING_TOOLS -> GENERATING ... -> TERMINATED.  Tokens produced by tools are appended
to the response with mask 0 so they never receive a policy gradient.
Parity target: ``verl/experimental/agent_loop/tool_agent_loop.py`` (states :48-52, loop :162-173, tools :298-506).
"""

from __future__ import annotations

import asyncio
import json
import time
from enum import Enum
from typing import Any, Optional
from uuid import uuid4

from ...tools.registry import initialize_tools_from_config
from ...tools.schemas import OpenAIFunctionCallSchema, OpenAIFunctionParsedSchema, ToolResponse
from .agent_loop import AgentLoopBase, AgentLoopMetrics, AgentLoopOutput, register
from .tool_parser import FunctionCall, ToolParser

__all__ = ["AgentState", "ToolAgentLoop"]


class AgentState(Enum):
    PENDING = "pending"
    GENERATING = "generating"
    PROCESSING_TOOLS = "processing_tools"
    TERMINATED = "terminated"


@register("tool_agent")
class ToolAgentLoop(AgentLoopBase):
    _tools_cache: dict[str, dict] = {}

    def __init__(self, trainer_config, server_manager, tokenizer=None, processor=None, tools: Optional[list] = None, **kwargs):
        super().__init__(trainer_config, server_manager, tokenizer, processor, **kwargs)
        mt = self.rollout_config.get("multi_turn") or {}
        self.max_user_turns = mt.get("max_user_turns")
        self.max_assistant_turns = mt.get("max_assistant_turns")
        self.max_parallel_calls = int(mt.get("max_parallel_calls", 1))
        self.max_tool_response_length = int(mt.get("max_tool_response_length", 256))
        self.truncate_side = mt.get("tool_response_truncate_side", "middle")
        path, fn_path = mt.get("tool_config_path"), mt.get("function_tool_path")
        if tools is None:
            if (path, fn_path) not in self._tools_cache:
                from ...tools.registry import load_all_tools

                self._tools_cache[(path, fn_path)] = {t.name: t for t in load_all_tools(path, fn_path)}
            self.tools = self._tools_cache[(path, fn_path)]
        else:
            self.tools = {t.name: t for t in tools}
        self.tool_schemas = [t.tool_schema.model_dump(exclude_unset=True, exclude_none=True) for t in self.tools.values()]
        self.parser = ToolParser.get_tool_parser(mt.get("format", "hermes"), tokenizer)
        self._ct_builder = None  # continuous-token builder, created on first use (False: template not supported)

    def _truncate(self, text: str) -> str:
        L = self.max_tool_response_length
        if len(text) <= L:
            return text
        if self.truncate_side == "left":
            return text[:L] + "...(truncated)"
        if self.truncate_side == "right":
            return "(truncated)..." + text[-L:]
        return text[: L // 2] + "...(truncated)..." + text[-L // 2:]

    async def _encode_tool_messages(self, messages: list[dict]) -> list[int]:
        """Token ids a chat template appends for tool messages + the next generation prompt (history is not
        re-tokenised: the ids are the difference against a rendering of a dummy system turn)."""
        tok = self.tokenizer
        if tok is None:
            text = "".join(f"\n<tool_response>{m['content']}</tool_response>" for m in messages) + "\n"
            return [ord(c) % 255 + 3 for c in text]
        if self._ct_builder is None and hasattr(tok, "encode") and hasattr(tok, "convert_tokens_to_ids"):
            from ...utils.tokenizer.continuous_token import build_continuous_token_builder

            try:
                self._ct_builder = build_continuous_token_builder(tok, getattr(tok, "name_or_path", None))
            except Exception:
                self._ct_builder = False  # template not prefix-stable for the synthetic base: plain difference below
        if self._ct_builder:
            return self._ct_builder.tokenize_non_assistant_incremental_messages(messages)
        base = tok.apply_chat_template([{"role": "system", "content": ""}], add_generation_prompt=False, tokenize=True)
        full = tok.apply_chat_template([{"role": "system", "content": ""}] + messages, add_generation_prompt=True, tokenize=True)
        return full[len(base):]

    async def _call_tool(self, call: FunctionCall, tools_kwargs: dict) -> tuple[ToolResponse, float]:
        tool, iid = None, None
        try:
            parsed, err = OpenAIFunctionCallSchema.from_openai_function_parsed_schema(
                OpenAIFunctionParsedSchema(name=call.name, arguments=call.arguments))
            if err:
                return ToolResponse(text="Error: tool arguments are not valid JSON"), 0.0
            tool = self.tools[parsed.name]
            kw = (tools_kwargs or {}).get(parsed.name, {})
            iid, _ = await tool.create(create_kwargs=kw.get("create_kwargs", {}))
            resp, reward, _ = await tool.execute(iid, parsed.arguments, **kw.get("execute_kwargs", {}))
            if resp.text:
                resp.text = self._truncate(resp.text)
            return resp, float(reward or 0.0)
        except KeyError:
            return ToolResponse(text=f"Error: unknown tool '{call.name}'"), 0.0
        except Exception as e:
            return ToolResponse(text=f"Error when executing tool: {e}"), 0.0
        finally:
            if tool is not None and iid is not None:
                await tool.release(iid)

    async def run(self, sampling_params: dict[str, Any], **kwargs) -> AgentLoopOutput:
        kwargs = dict(kwargs)
        kwargs.setdefault("tools", self.tool_schemas or None)
        prompt_ids = await self.prompt_ids_from(kwargs)
        rid = uuid4().hex
        m = AgentLoopMetrics()
        ids: list[int] = []
        mask: list[int] = []
        lps: list[float] = []
        state = AgentState.PENDING
        user_turns = assistant_turns = 0
        tool_rewards: list[float] = []
        calls: list[FunctionCall] = []
        while state != AgentState.TERMINATED:
            if state == AgentState.PENDING:
                state = AgentState.GENERATING
            elif state == AgentState.GENERATING:
                t0 = time.time()
                budget = self.response_length - len(ids)
                if budget <= 0:
                    state = AgentState.TERMINATED
                    continue
                out = await self.server_manager.generate(request_id=rid, prompt_ids=prompt_ids + ids,
                                                         sampling_params=dict(sampling_params, max_tokens=budget))
                m.generate_sequences += time.time() - t0
                assistant_turns += 1
                ids += out.token_ids
                mask += [1] * len(out.token_ids)
                lps += (out.log_probs or [0.0] * len(out.token_ids))
                if len(ids) >= self.response_length or (self.max_assistant_turns and assistant_turns >= self.max_assistant_turns) \
                        or (self.max_user_turns and user_turns >= self.max_user_turns):
                    state = AgentState.TERMINATED
                    continue
                _, calls = await self.parser.extract_tool_calls(out.token_ids)
                state = AgentState.PROCESSING_TOOLS if calls else AgentState.TERMINATED
            elif state == AgentState.PROCESSING_TOOLS:
                t0 = time.time()
                results = await asyncio.gather(*[self._call_tool(c, kwargs.get("tools_kwargs", {})) for c in calls[: self.max_parallel_calls]])
                m.tool_calls += time.time() - t0
                msgs = [{"role": "tool", "content": r.text or ""} for r, _ in results]
                tool_rewards += [rw for _, rw in results]
                tool_ids = await self._encode_tool_messages(msgs)
                if self._ct_builder:
                    # junction repair: close a turn that was cut without its end marker, do not repeat template text
                    merged = self._ct_builder.merge_non_assistant_tokens(prompt_ids + ids, tool_ids)
                    tool_ids = merged.token_ids[len(prompt_ids) + len(ids):]
                if len(ids) + len(tool_ids) >= self.response_length:
                    state = AgentState.TERMINATED
                    continue
                ids += tool_ids
                mask += [0] * len(tool_ids)
                lps += [0.0] * len(tool_ids)
                user_turns += 1
                state = AgentState.GENERATING
        ids, mask, lps = ids[: self.response_length], mask[: self.response_length], lps[: self.response_length]
        return AgentLoopOutput(prompt_ids=prompt_ids, response_ids=ids, response_mask=mask, response_logprobs=lps,
                               num_turns=user_turns + assistant_turns + 1, metrics=m,
                               extra_fields={"tool_rewards": tool_rewards} if tool_rewards else {})
