"""What a chat template adds around messages, found by probing the template rather than by knowing it.

Multi-turn rollouts build their token sequence piece by piece: the prompt, what the model generated, a tool or user turn
rendered on its own, more generation. Rendering a turn on its own repeats the template's default system prompt in front of
it and loses the separator the template puts between turns, so the pieces do not add up to ``apply_chat_template`` of the
whole conversation. These helpers recover the three constant pieces from a handful of probe renderings:

* ``initialize_system_prompt``: tokens the template puts in front of the first message (rendering one empty user turn and
  two of them differs by exactly one turn; what is left in front is the system part);
* ``initialize_turn_separator``: tokens between a message's closing token and the next turn (the common tail of two user
  turns that differ only in their text is ``[closing token, separator...]``; the model emits the closing token itself);
* ``extract_system_prompt_and_generation``: the system part and the generation prompt (what ``add_generation_prompt`` adds).

Parity target: ``verl/utils/tokenizer/chat_template.py:13-139``.
"""

from __future__ import annotations

from typing import Any

__all__ = ["normalize_token_ids", "initialize_system_prompt", "initialize_turn_separator", "extract_system_prompt_and_generation"]


def normalize_token_ids(out: Any) -> list[int]:
    """``apply_chat_template(tokenize=True)`` returns a list, a batch of one, a tensor or a dict with ``input_ids``."""
    if isinstance(out, dict) or hasattr(out, "input_ids"):
        out = out["input_ids"] if isinstance(out, dict) else out.input_ids
    if hasattr(out, "tolist"):
        out = out.tolist()
    out = list(out)
    if out and isinstance(out[0], (list, tuple)):
        assert len(out) == 1, "expected a single rendered conversation"
        out = list(out[0])
    return [int(t) for t in out]


def _render(tokenizer, messages, add_generation_prompt=False, **kw) -> list[int]:
    return normalize_token_ids(tokenizer.apply_chat_template(messages, add_generation_prompt=add_generation_prompt, tokenize=True, **kw))


def initialize_system_prompt(tokenizer, **apply_chat_template_kwargs) -> list[int]:
    one = _render(tokenizer, [{"role": "user", "content": ""}], **apply_chat_template_kwargs)
    two = _render(tokenizer, [{"role": "user", "content": ""}] * 2, **apply_chat_template_kwargs)
    turn = len(two) - len(one)
    return one[: len(one) - turn] if 0 < turn <= len(one) else []


def extract_system_prompt_and_generation(tokenizer, **apply_chat_template_kwargs) -> tuple[list[int], list[int]]:
    one = _render(tokenizer, [{"role": "user", "content": ""}], **apply_chat_template_kwargs)
    with_gen = _render(tokenizer, [{"role": "user", "content": ""}], add_generation_prompt=True, **apply_chat_template_kwargs)
    return initialize_system_prompt(tokenizer, **apply_chat_template_kwargs), with_gen[len(one):]


def initialize_turn_separator(tokenizer, **apply_chat_template_kwargs) -> list[int]:
    """Empty list when the template has no separator, or cannot be probed (callers then behave as before)."""
    empty = filled = None
    # some multi-modal processors reject a bare string body and want a list of typed parts: try both, same form for both probes
    for bodies in (("", "x"), ([{"type": "text", "text": ""}], [{"type": "text", "text": "x"}])):
        try:
            empty = _render(tokenizer, [{"role": "user", "content": bodies[0]}], **apply_chat_template_kwargs)
            filled = _render(tokenizer, [{"role": "user", "content": bodies[1]}], **apply_chat_template_kwargs)
            break
        except Exception:
            empty = filled = None
    if not empty or not filled:
        return []
    n = 0
    while n < len(empty) and n < len(filled) and empty[-1 - n] == filled[-1 - n]:
        n += 1
    tail = empty[len(empty) - n:]
    if not tail:
        return []
    eos = getattr(tokenizer, "eos_token_id", None)
    if eos is None:
        eos = getattr(getattr(tokenizer, "tokenizer", None), "eos_token_id", None)
    closing = {eos} if isinstance(eos, int) else set(eos or [])
    at = [i for i, t in enumerate(tail) if t in closing]
    return tail[at[-1] + 1:] if at else tail[1:]
