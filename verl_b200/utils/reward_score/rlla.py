"""Tool-use reward ("rlla" data): a format reward for the layout of the answer plus a graded reward for the tool calls.

The ground truth is itself a formatted answer: ``<think>...</think>`` followed by a ``<tool_call>`` block (one JSON object
``{"name": ..., "parameters": {...}}`` per line), a ``<response>`` block, both, or neither. The model's text is scored on

* format (0 or 1): it has exactly the blocks the ground truth has, in that order, each once, and nothing around them;
* tool calls (-3 .. 3; 0 when the ground truth calls no tool): exact equality of the parsed calls scores 3; otherwise
  partial credit is ``overlap of the tool names + for every expected call its best unused prediction of the same name
  (overlap of parameter names + number of parameters with the right value)``, divided by the most that could be had
  (``1 + sum over expected calls of (1 + number of parameters)``) and mapped linearly onto [-3, 3]. A prediction that
  cannot be parsed scores -3.

Overlap of two lists is the multiset Jaccard index (order ignored, multiplicity kept).

Parity target: ``verl/utils/reward_score/rlla.py`` (``match_score`` :21, ``customize_format_reward_func`` :44,
``compute_tool_call_reward`` :100, ``customize_correctness_reward_tool`` :155, ``compute_score`` :198).
"""

from __future__ import annotations

import json
import re
from collections import Counter

__all__ = ["match_score", "format_reward", "tool_call_reward", "correctness_reward", "assistant_text", "compute_score"]

TOOL_MAX, TOOL_MIN = 3.0, -3.0
_THINK = r"<think>.*?</think>"
_TOOL = r"<tool_call>\n.*?\n</tool_call>"
_RESP = r"<response>.*?</response>"


def match_score(a: list, b: list) -> float:
    """Multiset Jaccard index of two lists: 1 for equal lists, 0 when either is empty."""
    if a == b:
        return 1.0
    if not a or not b:
        return 0.0
    ca, cb = Counter(a), Counter(b)
    inter = sum((ca & cb).values())
    union = len(a) + len(b) - inter
    return inter / union if union > 0 else 0.0


def format_reward(response: str, answer: str, hi: float = 1.0, lo: float = 0.0) -> float:
    has_resp, has_tool = "<response>" in answer, "<tool_call>" in answer
    parts, once = [_THINK], []
    if has_tool:
        parts.append(_TOOL)
        once += ["<tool_call>", "</tool_call>"]
    if has_resp:
        parts.append(_RESP)
        once += ["<response>", "</response>"]
    ok = re.search("^" + r"\n".join(parts) + "$", response, re.DOTALL) is not None and all(response.count(t) == 1 for t in once)
    return hi if ok else lo


def tool_call_reward(expected: list[dict], predicted: list[dict], hi: float = TOOL_MAX, lo: float = TOOL_MIN) -> float:
    if expected == predicted:
        return hi
    score = match_score([t["name"] for t in expected], [t["name"] for t in predicted])
    best_possible = 1.0
    used: set[int] = set()
    for want in expected:
        params = want["parameters"]
        best_possible += 1.0 + len(params)
        best_i, best = -1, 0.0
        for i, got in enumerate(predicted):
            if i in used or got["name"] != want["name"]:
                continue
            gp = got["parameters"]
            s = match_score(list(params), list(gp)) + sum(1.0 for k, v in params.items() if k in gp and gp[k] == v)
            if s > best:
                best_i, best = i, s
        if best_i >= 0:
            used.add(best_i)
            score += best
    return (hi - lo) * score / best_possible + lo


def _calls(text: str) -> list[dict]:
    block = text.split("<tool_call>")[1].split("</tool_call>")[0].strip()
    return [json.loads(line) for line in block.split("\n")]


def correctness_reward(response: str, answer: str, hi: float = TOOL_MAX, lo: float = TOOL_MIN) -> float:
    if "<tool_call>" not in answer:
        return 0.0
    expected = _calls(answer)
    try:
        if "<tool_call>" not in response or "</tool_call>" not in response:
            return lo
        return tool_call_reward(expected, _calls(response), hi, lo)
    except Exception:
        return lo   # unparsable or malformed prediction: the lowest score, as a constraint on the format


def assistant_text(solution_str: str, experiment_name: str) -> str:
    """The last assistant turn of a decoded conversation, by the chat template the experiment's name points at."""
    name = experiment_name or ""
    if "llama" in name:
        return solution_str.split("<|start_header_id|>assistant<|end_header_id|>")[-1].split("<|eot_id|>")[0].strip()
    if "qwen" in name:
        return solution_str.split("<|im_start|>assistant")[-1].split("<|im_end|>")[0].strip()
    raise NotImplementedError(f"Unknown model name: {name}")


def compute_score(data_source, solution_str: str, ground_truth: str, extra_info=None, step: int = 0) -> dict:
    text = assistant_text(solution_str, (extra_info or {}).get("experiment_name", ""))
    fmt = format_reward(text, ground_truth)
    acc = correctness_reward(text, ground_truth)
    return {"score": fmt + acc, "format_reward": fmt, "accuracy_reward": acc}
