"""Tool-use reward: format and graded tool-call scores on hand-computed cases (semantics of verl/utils/reward_score/rlla.py)."""
import json

import pytest

from verl_b200.utils.reward_score import rlla


def _wrap(text):
    return f"<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n{text}<|im_end|>"


def _call(name, **params):
    return json.dumps({"name": name, "parameters": params})


def test_overlap_is_a_multiset_jaccard_index():
    assert rlla.match_score(["a", "b"], ["a", "b"]) == 1.0 and rlla.match_score([], ["a"]) == 0.0
    assert rlla.match_score(["a", "a", "b"], ["a", "c"]) == pytest.approx(1 / 4)     # one shared "a"; 3 + 2 - 1 = 4
    assert rlla.match_score(["a", "b"], ["b", "a"]) == 1.0                            # order is ignored


def test_format_reward_wants_exactly_the_blocks_of_the_ground_truth():
    tool = "<tool_call>\n" + _call("f", x=1) + "\n</tool_call>"
    gt_tool, gt_resp, gt_both, gt_none = f"<think>t</think>\n{tool}", "<think>t</think>\n<response>r</response>", \
        f"<think>t</think>\n{tool}\n<response>r</response>", "<think>t</think>"
    assert rlla.format_reward(f"<think>plan</think>\n{tool}", gt_tool) == 1.0
    assert rlla.format_reward(f"<think>plan</think>\n{tool}\n<response>x</response>", gt_tool) == 0.0      # a block too many
    assert rlla.format_reward(f"<think>plan</think>\n{tool}\n{tool}", gt_tool) == 0.0                       # the block twice
    assert rlla.format_reward("<think>a\nb</think>\n<response>fine</response>", gt_resp) == 1.0
    assert rlla.format_reward("hello <think>a</think>\n<response>fine</response>", gt_resp) == 0.0         # text in front
    assert rlla.format_reward(f"<think>p</think>\n{tool}\n<response>r</response>", gt_both) == 1.0
    assert rlla.format_reward(f"<think>p</think>\n<response>r</response>\n{tool}", gt_both) == 0.0         # wrong order
    assert rlla.format_reward("<think>only</think>", gt_none) == 1.0 and rlla.format_reward("no tags", gt_none) == 0.0


def test_tool_call_reward_gives_partial_credit():
    gt = [{"name": "search", "parameters": {"q": "cats", "k": 3}}, {"name": "open", "parameters": {"url": "u"}}]
    assert rlla.tool_call_reward(gt, [dict(t) for t in gt]) == 3.0
    # best possible = 1 + (1 + 2) + (1 + 1) = 6. Prediction: only "search" with q right, k wrong:
    # names overlap 1/2; parameter names overlap 1, one right value -> 0.5 + 2 = 2.5 -> 6 * 2.5 / 6 - 3 = -0.5
    pd = [{"name": "search", "parameters": {"q": "cats", "k": 5}}]
    assert rlla.tool_call_reward(gt, pd) == pytest.approx(-0.5)
    # nothing in common: names overlap 0, no match -> the minimum
    assert rlla.tool_call_reward(gt, [{"name": "other", "parameters": {}}]) == -3.0
    # a prediction is used for one expected call only: two expected "f" calls, one predicted
    gt2 = [{"name": "f", "parameters": {"a": 1}}, {"name": "f", "parameters": {"a": 1}}]
    pd2 = [{"name": "f", "parameters": {"a": 1}}]
    # best possible 1 + 2 + 2 = 5; names overlap 1/2; the first expected call takes the prediction (1 + 1) -> 2.5 -> 6*2.5/5-3 = 0
    assert rlla.tool_call_reward(gt2, pd2) == pytest.approx(0.0)


def test_compute_score_adds_the_two_parts_and_punishes_unparsable_calls():
    tool = "<tool_call>\n" + _call("search", q="cats") + "\n</tool_call>"
    gt = f"<think>t</think>\n{tool}"
    info = {"experiment_name": "qwen2.5-tooluse"}
    good = rlla.compute_score("rlla", _wrap(f"<think>I search</think>\n{tool}"), gt, info)
    assert good == {"score": 4.0, "format_reward": 1.0, "accuracy_reward": 3.0}
    broken = rlla.compute_score("rlla", _wrap("<think>x</think>\n<tool_call>\nnot json\n</tool_call>"), gt, info)
    assert broken["format_reward"] == 1.0 and broken["accuracy_reward"] == -3.0 and broken["score"] == -2.0
    missing = rlla.compute_score("rlla", _wrap("<think>x</think>\n<response>no tool</response>"), gt, info)
    assert missing["format_reward"] == 0.0 and missing["accuracy_reward"] == -3.0
    no_tool_gt = rlla.compute_score("rlla", _wrap("<think>x</think>\n<response>hi</response>"), "<think>t</think>\n<response>r</response>", info)
    assert no_tool_gt == {"score": 1.0, "format_reward": 1.0, "accuracy_reward": 0.0}
    llama = "<|start_header_id|>assistant<|end_header_id|>\n\n<think>x</think>\n<response>hi</response><|eot_id|>"
    assert rlla.compute_score("rlla", llama, "<think>t</think>\n<response>r</response>", {"experiment_name": "llama3"})["score"] == 1.0
    with pytest.raises(NotImplementedError):
        rlla.compute_score("rlla", "x", gt, {"experiment_name": "mistral"})
