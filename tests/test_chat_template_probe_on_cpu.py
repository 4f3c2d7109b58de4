"""Constant pieces of a chat template recovered by probing it (a small ChatML-like template with a default system prompt)."""
import torch

from verl_b200.utils.tokenizer.chat_template import (extract_system_prompt_and_generation, initialize_system_prompt,
                                                     initialize_turn_separator, normalize_token_ids)

BOS, IM_START, IM_END, NL, SYS, USER, ASSISTANT, DEFAULT = 1, 10, 11, 12, 20, 21, 22, 30


class _ChatML:
    """<bos> [<im_start>system\\n DEFAULT <im_end>\\n] (<im_start>role\\n body <im_end>\\n)* [<im_start>assistant\\n]"""

    eos_token_id = IM_END

    def __init__(self, default_system=True, separator=True, parts_only=False, as_tensor=False):
        self.default_system, self.separator, self.parts_only, self.as_tensor = default_system, separator, parts_only, as_tensor

    def apply_chat_template(self, messages, add_generation_prompt=False, tokenize=True, **kw):
        role_id = {"system": SYS, "user": USER, "assistant": ASSISTANT}
        out = [BOS]
        if self.default_system and not (messages and messages[0]["role"] == "system"):
            out += [IM_START, SYS, NL, DEFAULT, IM_END] + ([NL] if self.separator else [])
        for m in messages:
            body = m["content"]
            if self.parts_only and isinstance(body, str):
                raise TypeError("content must be a list of parts")
            text = body if isinstance(body, str) else "".join(p["text"] for p in body)
            out += [IM_START, role_id[m["role"]], NL] + [100 + ord(c) for c in text] + [IM_END] + ([NL] if self.separator else [])
        if add_generation_prompt:
            out += [IM_START, ASSISTANT, NL]
        return {"input_ids": torch.tensor([out])} if self.as_tensor else out


def test_pieces_of_a_template_with_a_default_system_prompt():
    tok = _ChatML()
    assert initialize_system_prompt(tok) == [BOS, IM_START, SYS, NL, DEFAULT, IM_END, NL]
    assert extract_system_prompt_and_generation(tok) == ([BOS, IM_START, SYS, NL, DEFAULT, IM_END, NL], [IM_START, ASSISTANT, NL])
    assert initialize_turn_separator(tok) == [NL]
    # pieces add up: prompt + generated + separator + (tool turn rendered alone, minus the system part) == whole conversation
    user = [{"role": "user", "content": "hi"}]
    reply = [100 + ord("o"), 100 + ord("k"), IM_END]       # what the model emits, closing token included
    tool = [{"role": "user", "content": "t"}]
    prompt = tok.apply_chat_template(user, add_generation_prompt=True)
    alone = tok.apply_chat_template(tool, add_generation_prompt=True)[len(initialize_system_prompt(tok)):]
    whole = tok.apply_chat_template(user + [{"role": "assistant", "content": "ok"}] + tool, add_generation_prompt=True)
    assert prompt + reply + initialize_turn_separator(tok) + alone == whole


def test_templates_without_system_part_or_separator_and_odd_return_types():
    assert initialize_system_prompt(_ChatML(default_system=False)) == [BOS]
    assert initialize_turn_separator(_ChatML(separator=False)) == []
    assert initialize_turn_separator(_ChatML(parts_only=True)) == [NL]          # falls back to the list-of-parts body
    assert initialize_turn_separator(_ChatML(as_tensor=True)) == [NL]            # dict of a batched tensor
    assert normalize_token_ids(torch.tensor([[3, 4]])) == [3, 4] and normalize_token_ids({"input_ids": [5, 6]}) == [5, 6]

    class Broken:
        eos_token_id = None

        def apply_chat_template(self, *a, **k):
            raise RuntimeError("no template")

    assert initialize_turn_separator(Broken()) == []
