"""Continuous-token builder on a toy ChatML-style tokenizer whose text tokenisation is context dependent (so that
re-rendering history would change earlier tokens, which the builder must never do)."""
import pytest

from verl_b200.utils.tokenizer.continuous_token import ContinuousTokenBuilder, build_continuous_token_builder

IM_START, IM_END, NL = 1, 2, 3


class ToyTokenizer:
    """``<|im_start|>role\\ncontent<|im_end|>\\n`` per message; words map to ids, and a word directly after "the" gets a
    different id than elsewhere (a stand-in for merges across boundaries in real BPE vocabularies)."""

    def __init__(self):
        self.vocab = {"<|im_start|>": IM_START, "<|im_end|>": IM_END, "\n": NL}

    def get_vocab(self):
        return dict(self.vocab)

    def convert_tokens_to_ids(self, toks):
        return [self.vocab[t] for t in toks]

    def _word(self, w, prev):
        key = ("after_the:" + w) if prev == "the" else w
        return self.vocab.setdefault(key, len(self.vocab) + 10)

    def encode(self, text, add_special_tokens=False):
        out, prev = [], None
        for w in text.split():
            out.append(self._word(w, prev))
            prev = w
        return out

    def apply_chat_template(self, messages, tools=None, add_generation_prompt=False, tokenize=True, **kw):
        ids = []
        for m in messages:
            ids += [IM_START] + self.encode(m["role"]) + [NL] + self.encode(str(m["content"])) + [IM_END, NL]
        if add_generation_prompt:
            ids += [IM_START] + self.encode("assistant") + [NL]
        return ids


def test_multi_turn_stream_only_grows_and_matches_a_full_rendering():
    tok = ToyTokenizer()
    b = ContinuousTokenBuilder(tok)
    assert b.eot_ids == [IM_END, NL]
    msgs = [{"role": "user", "content": "what is the answer"}]
    run = b.build_initial_tokens(msgs)
    # the model samples an assistant turn that ends with <|im_end|> (no newline: that is template text)
    sampled = tok.encode("call the tool") + [IM_END]
    r1 = b.merge_assistant_tokens(run, sampled)
    assert r1.kind == "assistant" and r1.appended_token_count == len(sampled) and r1.token_ids[: len(run)] == run
    inc = b.tokenize_non_assistant_incremental_messages([{"role": "tool", "content": "the result is 42"}])
    r2 = b.merge_non_assistant_tokens(r1.token_ids, inc)
    assert r2.inserted_token_ids == [NL] and r2.removed_prefix_token_count == 0
    assert r2.token_ids[: len(r1.token_ids)] == r1.token_ids          # history untouched
    full = tok.apply_chat_template(msgs + [{"role": "assistant", "content": "call the tool"}, {"role": "tool", "content": "the result is 42"}],
                                   add_generation_prompt=True)
    assert r2.token_ids == full
    mask, lps = b.align_response_metadata(r1, [], [], assistant_logprobs=[-0.1] * len(sampled))
    mask, lps = b.align_response_metadata(r2, mask, lps)
    assert len(mask) == len(r2.token_ids) - len(run) == len(lps)
    assert mask[: len(sampled)] == [1] * len(sampled) and set(mask[len(sampled):]) == {0} and lps[len(sampled)] == 0.0


def test_length_cut_turn_gets_the_end_marker_and_bad_roles_are_rejected():
    tok = ToyTokenizer()
    b = build_continuous_token_builder(tok, model_type="qwen2")
    run = b.build_initial_tokens([{"role": "user", "content": "hi"}])
    cut = tok.encode("an unfinished")                                   # stopped by the length limit: no <|im_end|>
    r1 = b.merge_assistant_tokens(run, cut)
    inc = b.tokenize_non_assistant_incremental_messages([{"role": "user", "content": "go on"}])
    r2 = b.merge_non_assistant_tokens(r1.token_ids, inc)
    assert r2.inserted_token_ids == [IM_END, NL]
    assert r2.token_ids == r1.token_ids + [IM_END, NL] + inc
    with pytest.raises(ValueError):
        b.tokenize_non_assistant_incremental_messages([{"role": "assistant", "content": "x"}])


def test_async_rollout_request_tracks_tokens_masks_and_states():
    from verl_b200.workers.rollout.schemas import AsyncRolloutRequest, AsyncRolloutRequestStateEnum, FinishReasonTypeEnum

    tok = ToyTokenizer()
    req = AsyncRolloutRequest.create("r1", [{"role": "user", "content": "what is the answer"}], tok, max_response_len=64)
    n0 = len(req.input_ids)
    assert req.state == AsyncRolloutRequestStateEnum.PENDING and req.loss_mask == [0] * n0 and req.response_ids == []
    sampled = tok.encode("call the tool") + [IM_END]
    req.add_assistant_message("call the tool", sampled, logprobs=[-0.5] * len(sampled), tool_calls=[{"name": "calc"}])
    assert req.state == AsyncRolloutRequestStateEnum.TOOL_CALLING and req.response_loss_mask == [1] * len(sampled)
    req.add_tool_response_messages(["the result is 42"])
    assert req.state == AsyncRolloutRequestStateEnum.RUNNING
    full = tok.apply_chat_template([{"role": "user", "content": "what is the answer"}, {"role": "assistant", "content": "call the tool"},
                                    {"role": "tool", "content": "the result is 42"}], add_generation_prompt=True)
    assert req.input_ids == full and req.get_generation_prompt_ids() == full
    assert sum(req.response_loss_mask) == len(sampled) and len(req.response_loss_mask) == len(full) - n0
    final = tok.encode("42") + [IM_END]
    req.add_assistant_message("42", final)
    req.max_response_len = len(req.response_ids) - 1          # force a truncation by one token
    req.finalize({"score": 1.0}, FinishReasonTypeEnum.from_str("stop"))
    assert req.state == AsyncRolloutRequestStateEnum.COMPLETED and len(req.response_ids) == req.max_response_len
    assert len(req.input_ids) == len(req.loss_mask) == n0 + req.max_response_len and req.reward_scores == {"score": 1.0}
