"""Exact-match / sub-string-match QA scoring on the last ``<answer>...</answer>`` span.

Parity target: ``verl/utils/reward_score/search_r1_like_qa_em.py`` (normalisation :23-37, EM :40, sub-EM :53,
answer-tag spam penalty score/4 :118-121).
"""

from __future__ import annotations

import re
import string

__all__ = ["normalize_answer", "em_check", "subem_check", "extract_solution", "compute_score", "compute_score_subem"]

_ARTICLES = re.compile(r"\b(a|an|the)\b")
_PUNCT = str.maketrans("", "", string.punctuation)


def normalize_answer(s: str) -> str:
    s = _ARTICLES.sub(" ", str(s).lower().translate(_PUNCT))
    return " ".join(s.split())


def _targets(golden) -> list[str]:
    if isinstance(golden, str):
        golden = [golden]
    return [normalize_answer(g) for g in list(golden)]


def em_check(prediction: str, golden_answers) -> int:
    p = normalize_answer(prediction)
    return int(any(g == p for g in _targets(golden_answers)))


def subem_check(prediction: str, golden_answers) -> int:
    p = normalize_answer(prediction)
    return int(any(g in p for g in _targets(golden_answers)))


def extract_solution(solution_str: str):
    found = re.findall(r"<answer>(.*?)</answer>", solution_str, re.DOTALL)
    return found[-1].strip() if found else None


def _score(solution_str, ground_truth, check, format_score, score):
    answer = extract_solution(solution_str)
    if answer is None:
        return 0
    target = ground_truth["target"] if isinstance(ground_truth, dict) else ground_truth
    if not check(answer, target):
        return format_score
    spam = solution_str.count("<answer>") > 10 or solution_str.count("</answer>") > 10
    return score / 4 if spam else score


def compute_score(solution_str, ground_truth, method="strict", format_score=0.0, score=1.0):
    return _score(solution_str, ground_truth, em_check, format_score, score)


def compute_score_subem(solution_str, ground_truth, method="strict", format_score=0.0, score=1.0):
    return _score(solution_str, ground_truth, subem_check, format_score, score)
