"""Request state of a multi-turn (tool-using) rollout: the message list, the token stream with its masks, and the
transitions between pending / running / tool-calling / finished.

The token stream only grows: assistant turns are appended as the sampled ids (loss mask 1), user / tool turns through the
continuous-token builder (loss mask 0), so what the trainer sees is exactly what the model saw.
Parity target: ``verl/workers/rollout/schemas.py`` (``FinishReasonTypeEnum`` :38, ``Message`` :57,
``AsyncRolloutRequestStateEnum`` :63, ``AsyncRolloutRequest`` :81 with ``get_generation_prompt_ids`` :374,
``add_user_message`` :406, ``add_assistant_message`` :428, ``add_tool_response_messages`` :453, ``finalize`` :591,
``truncate_output_ids`` :699).
"""

from __future__ import annotations

from enum import Enum
from typing import Any, Optional

from pydantic import BaseModel, ConfigDict, Field

__all__ = ["FinishReasonTypeEnum", "Message", "AsyncRolloutRequestStateEnum", "TokenizationSanityCheckModeEnum", "AsyncRolloutRequest"]


class FinishReasonTypeEnum(str, Enum):
    LENGTH = "length"
    STOP = "stop"
    TOOL_CALL = "tool_calls"

    @classmethod
    def from_str(cls, value: str) -> "FinishReasonTypeEnum":
        v = (value or "").lower()
        if v in ("length", "max_tokens"):
            return cls.LENGTH
        if v in ("stop", "completed", "eos"):
            return cls.STOP
        if v in ("tool_calls", "tool_call"):
            return cls.TOOL_CALL
        raise ValueError(f"unknown finish reason {value!r}")


class Message(BaseModel):
    role: str
    content: Any = ""
    tool_calls: Optional[list] = None


class AsyncRolloutRequestStateEnum(str, Enum):
    PENDING = "pending"
    RUNNING = "running"
    COMPLETED = "completed"
    FAILED = "failed"
    TOOL_CALLING = "tool_calling"
    INTERACTING = "interacting"


class TokenizationSanityCheckModeEnum(str, Enum):
    DISABLE = "disable"
    STRICT = "strict"
    IGNORE_STRIPPABLE = "ignore_strippable"


class AsyncRolloutRequest(BaseModel):
    model_config = ConfigDict(arbitrary_types_allowed=True)

    batch_data_id: int = 0
    rollout_offset: int = 0
    request_id: str
    state: AsyncRolloutRequestStateEnum = AsyncRolloutRequestStateEnum.PENDING
    messages: list[Message]
    tool_schemas: Optional[list] = None
    tools_kwargs: dict = Field(default_factory=dict)
    input_ids: list[int] = Field(default_factory=list)
    prompt_ids: list[int] = Field(default_factory=list)
    response_ids: list[int] = Field(default_factory=list)
    attention_mask: list[int] = Field(default_factory=list)
    loss_mask: list[int] = Field(default_factory=list)
    response_loss_mask: list[int] = Field(default_factory=list)
    response_logprobs: list[float] = Field(default_factory=list)
    reward_scores: dict = Field(default_factory=dict)
    metrics: dict = Field(default_factory=dict)
    max_prompt_len: int = 1 << 30
    max_response_len: int = 8192
    max_model_len: int = 32768
    builder: Any = Field(default=None, exclude=True)   # ContinuousTokenBuilder

    # ---- construction
    @classmethod
    def create(cls, request_id: str, messages: list, tokenizer, tools: Optional[list] = None, **kwargs) -> "AsyncRolloutRequest":
        from ...utils.tokenizer.continuous_token import build_continuous_token_builder

        msgs = [m if isinstance(m, Message) else Message(**m) for m in messages]
        builder = build_continuous_token_builder(tokenizer, getattr(tokenizer, "name_or_path", None), tools=tools)
        ids = builder.build_initial_tokens([m.model_dump(exclude_none=True) for m in msgs])
        req = cls(request_id=request_id, messages=msgs, tool_schemas=tools, builder=builder, **kwargs)
        if len(ids) > req.max_prompt_len:
            ids = ids[-req.max_prompt_len:]  # keep the end of the prompt (the generation prompt must survive)
        req.input_ids, req.prompt_ids = list(ids), list(ids)
        req.attention_mask, req.loss_mask = [1] * len(ids), [0] * len(ids)
        return req

    # ---- queries
    def get_generation_prompt_ids(self) -> list[int]:
        return list(self.input_ids)

    @property
    def remaining_response_tokens(self) -> int:
        return max(0, min(self.max_response_len - len(self.response_ids), self.max_model_len - len(self.input_ids)))

    # ---- transitions
    def _extend(self, ids: list[int], mask: int, logprobs: Optional[list[float]] = None) -> None:
        self.input_ids += ids
        self.response_ids += ids
        self.attention_mask += [1] * len(ids)
        self.loss_mask += [mask] * len(ids)
        self.response_loss_mask += [mask] * len(ids)
        self.response_logprobs += list(logprobs) if logprobs is not None else [0.0] * len(ids)

    def add_assistant_message(self, content: str, token_ids: list[int], logprobs: Optional[list[float]] = None,
                              tool_calls: Optional[list] = None) -> None:
        """The sampled ids are appended as they are (never re-tokenised)."""
        self.messages.append(Message(role="assistant", content=content, tool_calls=tool_calls))
        self._extend(list(token_ids), 1, logprobs)
        self.state = AsyncRolloutRequestStateEnum.TOOL_CALLING if tool_calls else AsyncRolloutRequestStateEnum.RUNNING

    def _add_non_assistant(self, new: list[Message]) -> None:
        self.messages += new
        inc = self.builder.tokenize_non_assistant_incremental_messages([m.model_dump(exclude_none=True) for m in new])
        merged = self.builder.merge_non_assistant_tokens(self.input_ids, inc)
        self._extend(merged.token_ids[len(self.input_ids):], 0)

    def add_user_message(self, content: str) -> None:
        self._add_non_assistant([Message(role="user", content=content)])
        self.state = AsyncRolloutRequestStateEnum.RUNNING

    def add_tool_response_messages(self, contents: list) -> None:
        self._add_non_assistant([Message(role="tool", content=c) for c in contents])
        self.state = AsyncRolloutRequestStateEnum.RUNNING

    def update_metrics(self, metrics: Any, tool_id: str) -> None:
        self.metrics.setdefault(tool_id, []).append(metrics)

    def truncate_output_ids(self) -> None:
        over = len(self.response_ids) - self.max_response_len
        over = max(over, len(self.input_ids) - self.max_model_len)
        if over > 0:
            for name in ("input_ids", "attention_mask", "loss_mask", "response_ids", "response_loss_mask", "response_logprobs"):
                setattr(self, name, getattr(self, name)[:-over])

    def finalize(self, reward_scores: Optional[dict] = None, finish_reason: FinishReasonTypeEnum = FinishReasonTypeEnum.STOP) -> None:
        self.state = AsyncRolloutRequestStateEnum.COMPLETED
        if reward_scores:
            self.reward_scores.update(reward_scores)
        self.metrics["finish_reason"] = finish_reason.value
        self.truncate_output_ids()
        assert len(self.input_ids) == len(self.attention_mask) == len(self.loss_mask)
        assert len(self.response_ids) == len(self.response_loss_mask) == len(self.response_logprobs)
