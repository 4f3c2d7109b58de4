"""Rule-based scoring functions keyed by ``data_source``.

Parity target: ``verl/utils/reward_score/__init__.py:19`` (``default_compute_score``) and its per-dataset modules.
"""

from __future__ import annotations

__all__ = ["default_compute_score"]


def default_compute_score(data_source, solution_str, ground_truth, extra_info=None, sandbox_fusion_url=None,
                          concurrent_semaphore=None, memory_limit_mb=None, **kwargs):
    src = str(data_source)
    if src == "openai/gsm8k":
        from . import gsm8k

        res = gsm8k.compute_score(solution_str, ground_truth)
    elif src in ("lighteval/MATH", "DigitalLearningGmbH/MATH-lighteval", "HuggingFaceH4/MATH-500"):
        from . import math_reward

        res = math_reward.compute_score(solution_str, ground_truth)
    elif src in ("math_dapo", "math", "math_dapo_reasoning") or src.startswith("aime"):
        from . import math_dapo

        res = math_dapo.compute_score(solution_str, ground_truth)
    elif src in ("numina_aops_forum", "numina_synthetic_math", "numina_amc_aime", "numina_synthetic_amc",
                 "numina_cn_k12", "numina_olympiads"):
        from . import prime_math

        res = prime_math.compute_score(solution_str, ground_truth)
    elif src in ("codecontests", "apps", "codeforces", "taco"):
        from . import prime_code

        res = prime_code.compute_score(solution_str, ground_truth, continuous=True)
    elif src == "hiyouga/geometry3k":
        from . import geo3k

        res = geo3k.compute_score(solution_str, ground_truth)
    elif src.startswith("searchR1_") or src in ("nq", "triviaqa", "popqa", "hotpotqa", "2wikimultihopqa", "musique", "bamboogle"):
        from . import search_r1_like_qa_em

        res = search_r1_like_qa_em.compute_score(solution_str, ground_truth)
    elif src.startswith("synthetic/"):
        from . import synthetic

        res = synthetic.compute_score(solution_str, ground_truth, extra_info)
    else:
        raise NotImplementedError(f"Reward function is not implemented for {data_source=}")
    if isinstance(res, dict):
        return res
    if isinstance(res, (int, float, bool)):
        return float(res)
    return float(res[0])
