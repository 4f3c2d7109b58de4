"""Continuous-token prompts for multi-turn rollouts: the token stream the model saw and produced is kept as is and only
grows. New tool / user / system messages are tokenised incrementally (never by re-rendering the history, which can
re-tokenise earlier assistant text differently from what was sampled), assistant turns are appended as the sampled ids.

Incremental tokens of appended messages = rendering of (synthetic base + appended messages, with generation prompt) minus
the rendering of the synthetic base: chat templates are prefix-stable for appended turns, so the difference is exactly
what the template would add after a finished assistant turn. At the junction the builder repairs two cases: an assistant
turn that stopped without the end-of-turn marker (length cut) gets the marker inserted, and template text that the model
already produced (e.g. a trailing newline after the marker) is not inserted twice. Inserted boundary tokens are not
model output: ``align_response_metadata`` gives them mask 0 and log-prob 0.

Parity target: ``verl/utils/tokenizer/continuous_token.py`` (``MergeResult`` :37, ``ContinuousTokenBuilder`` :56 with
``build_initial_tokens`` :97, ``tokenize_non_assistant_incremental_messages`` :109, ``merge_non_assistant_tokens`` :145,
``merge_assistant_tokens`` :158, ``align_response_metadata`` :308) and ``continuous_token_wiring.py`` (builder selection).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Literal, Optional

__all__ = ["MergeResult", "ContinuousTokenBuilder", "build_continuous_token_builder"]

MergeKind = Literal["assistant", "non_assistant"]
_APPEND_ROLES = frozenset({"tool", "user", "system"})
_BASE = [{"role": "system", "content": "continuous token synthetic system"},
         {"role": "user", "content": "continuous token synthetic user"},
         {"role": "assistant", "content": "continuous token synthetic assistant"}]


@dataclass(frozen=True)
class MergeResult:
    """The updated stream and how it changed at the junction: ``inserted_token_ids`` were created by the builder (not by
    the model), ``appended_token_count`` counts the newly appended tokens without them, ``removed_prefix_token_count``
    tokens of the increment were dropped because the stream already ended with them."""

    token_ids: list[int]
    appended_token_count: int
    kind: MergeKind = "non_assistant"
    inserted_token_ids: list[int] = field(default_factory=list)
    removed_prefix_token_count: int = 0


class ContinuousTokenBuilder:
    def __init__(self, tokenizer: Any, tools: Optional[list[dict]] = None, chat_template_kwargs: Optional[dict] = None,
                 end_of_turn_token: Optional[str] = None):
        self.tokenizer = tokenizer
        self.tools = tools
        self.kw = dict(chat_template_kwargs or {})
        self._base_ids: Optional[list[int]] = None
        self.eot_ids = self._end_of_turn_ids(end_of_turn_token)

    # ---- rendering
    def _render(self, messages: list[dict], add_generation_prompt: bool) -> list[int]:
        out = self.tokenizer.apply_chat_template(messages, tools=self.tools, add_generation_prompt=add_generation_prompt,
                                                 tokenize=True, **self.kw)
        if isinstance(out, dict):
            out = out["input_ids"]
        return [int(t) for t in out]

    def _base(self) -> list[int]:
        if self._base_ids is None:
            self._base_ids = self._render(_BASE, add_generation_prompt=False)
        return self._base_ids

    def _end_of_turn_ids(self, token: Optional[str]) -> list[int]:
        """Ids that close an assistant turn in this template: what follows the assistant text in a rendering."""
        if token is not None:
            ids = self.tokenizer.convert_tokens_to_ids([token])
            return [int(i) for i in ids]
        probe = "continuous token synthetic assistant"
        enc = getattr(self.tokenizer, "encode", None)
        if enc is None:
            return []
        text_ids = [int(t) for t in enc(probe, add_special_tokens=False)]
        base = self._base()
        # last occurrence of the assistant text inside the rendered base; the tail after it is the closing sequence
        for s in range(len(base) - len(text_ids), -1, -1):
            if base[s : s + len(text_ids)] == text_ids:
                return base[s + len(text_ids) :]
        return []

    # ---- API
    def build_initial_tokens(self, messages: list[dict]) -> list[int]:
        return self._render(messages, add_generation_prompt=True)

    def tokenize_non_assistant_incremental_messages(self, appended_messages: list[dict]) -> list[int]:
        for m in appended_messages:
            if m.get("role") not in _APPEND_ROLES:
                raise ValueError(f"only {sorted(_APPEND_ROLES)} messages can be appended incrementally, got {m.get('role')!r}")
        base = self._base()
        full = self._render(_BASE + list(appended_messages), add_generation_prompt=True)
        if full[: len(base)] != base:
            raise ValueError("the chat template is not prefix-stable for appended messages; a model-specific builder is needed")
        return full[len(base) :]

    def merge_assistant_tokens(self, runtime_token_ids: list[int], assistant_token_ids: list[int]) -> MergeResult:
        return MergeResult(list(runtime_token_ids) + list(assistant_token_ids), len(assistant_token_ids), kind="assistant")

    def merge_non_assistant_tokens(self, runtime_token_ids: list[int], incremental_token_ids: list[int]) -> MergeResult:
        run, inc = list(runtime_token_ids), list(incremental_token_ids)
        eot = self.eot_ids
        inserted: list[int] = []
        removed = 0
        if eot:
            # how much of the closing sequence does the stream already end with? (the model usually samples its first token,
            # the template may add more, e.g. a newline)
            have = 0
            for n in range(len(eot), 0, -1):
                if run[-n:] == eot[:n]:
                    have = n
                    break
            inserted = eot[have:]
        # template text the stream (plus the inserted closing) already ends with is not appended twice
        tail = run + inserted
        for n in range(min(len(inc), len(tail)), 0, -1):
            if tail[-n:] == inc[:n] and n <= len(inserted):
                removed = n
                break
        new = inserted + inc[removed:]
        return MergeResult(run + new, len(inc) - removed, kind="non_assistant", inserted_token_ids=inserted,
                           removed_prefix_token_count=removed)

    @staticmethod
    def align_response_metadata(result: MergeResult, response_mask: list[int], response_logprobs: Optional[list[float]] = None,
                                assistant_logprobs: Optional[list[float]] = None):
        """Extend the per-token mask / log-prob lists of the response by what ``result`` added: sampled assistant tokens
        carry mask 1 and their log-probs, everything else (boundary tokens, tool / user text) mask 0 and log-prob 0."""
        n_ins, n_app = len(result.inserted_token_ids), result.appended_token_count
        mask = list(response_mask) + [0] * n_ins + [1 if result.kind == "assistant" else 0] * n_app
        if response_logprobs is None:
            return mask, None
        if result.kind == "assistant":
            lp = list(assistant_logprobs) if assistant_logprobs is not None else [0.0] * n_app
            assert len(lp) == n_app, "one log-prob per sampled token"
        else:
            lp = [0.0] * n_app
        return mask, list(response_logprobs) + [0.0] * n_ins + lp


def build_continuous_token_builder(tokenizer: Any, model_type: Optional[str] = None, **kwargs) -> ContinuousTokenBuilder:
    """Builder for a tokenizer / model family. Families whose templates close a turn with more than the sampled end token
    (ChatML: ``<|im_end|>`` + newline) are handled by the generic junction repair; the end-of-turn marker can be named
    explicitly for templates where it cannot be inferred."""
    eot = kwargs.pop("end_of_turn_token", None)
    if eot is None and model_type and any(k in model_type.lower() for k in ("qwen", "chatml")):
        vocab = getattr(tokenizer, "get_vocab", lambda: {})()
        eot = "<|im_end|>" if "<|im_end|>" in vocab else None
        if eot is not None:
            b = ContinuousTokenBuilder(tokenizer, **kwargs)
            nl = b._end_of_turn_ids(None)
            if nl and nl[0] == tokenizer.convert_tokens_to_ids([eot])[0]:
                return b  # inferred closing sequence already starts with the marker (and keeps what follows it)
    return ContinuousTokenBuilder(tokenizer, end_of_turn_token=eot, **kwargs)
