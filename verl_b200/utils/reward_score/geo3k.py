"""Geometry3K: 0.9 x boxed-answer accuracy + 0.1 x ``<think>..</think>..\\boxed{}`` format reward.

Parity target: ``verl/utils/reward_score/geo3k.py:20-36`` (the reference grades with an external ``mathruler``
package; here the grader is this package's own answer normaliser).
"""

from __future__ import annotations

import re

from .math_reward import is_equiv, last_boxed_only_string, remove_boxed

_FORMAT = re.compile(r"<think>.*</think>.*\\boxed\{.*\}.*", re.DOTALL)


def format_reward(predict_str: str) -> float:
    return 1.0 if _FORMAT.fullmatch(predict_str) else 0.0


def acc_reward(predict_str: str, ground_truth: str, use_boxed: bool = True) -> float:
    answer = predict_str
    if use_boxed:
        boxed = last_boxed_only_string(predict_str)
        if boxed is None:
            return 0.0
        answer = remove_boxed(boxed)
    return 1.0 if is_equiv(answer, str(ground_truth)) else 0.0


def compute_score(predict_str: str, ground_truth: str, use_boxed: bool = True, format_score: float = 0.1) -> float:
    return (1.0 - format_score) * acc_reward(predict_str, ground_truth, use_boxed) + format_score * format_reward(predict_str)
