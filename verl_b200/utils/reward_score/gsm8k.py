"""GSM8K: the final answer after '####' (strict) or the last number in the text (flexible)."""

import re

_STRICT = re.compile(r"#### (\-?[0-9\.\,]+)")
_NUMBER = re.compile(r"(\-?[0-9\.\,]+)")


def extract_solution(solution_str: str, method: str = "strict"):
    assert method in ("strict", "flexible")
    text = solution_str[-300:] if len(solution_str) > 300 else solution_str
    if method == "strict":
        hits = _STRICT.findall(text)
        return hits[-1].replace(",", "").replace("$", "") if hits else None
    for cand in reversed(_NUMBER.findall(text)):
        if cand not in ("", "."):
            return cand
    return None


def compute_score(solution_str: str, ground_truth: str, method: str = "strict", format_score: float = 0.0, score: float = 1.0):
    ans = extract_solution(solution_str, method)
    if ans is None:
        return 0.0
    return score if ans == str(ground_truth) else format_score
