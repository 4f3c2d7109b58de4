"""Batched wrapper of the MATH scorer. Parity target: ``verl/utils/reward_score/math_batch.py:18``."""
from .math_reward import compute_score


def compute_score_batched(data_sources, solution_strs, ground_truths, extra_infos=None):
    return [compute_score(s, g) for s, g in zip(solution_strs, ground_truths)]
