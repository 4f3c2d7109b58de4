"""Answer verification with a wall-clock limit: the comparison runs in a worker process so that a pathological
expression cannot stall the trainer; a timeout yields ``timeout_score``.

Parity target: ``verl/utils/reward_score/math_verify.py:33-67`` (the reference delegates to the external
``math_verify`` package; this build verifies with ``prime_math.grade_answer``).
"""

from __future__ import annotations

import concurrent.futures as cf

_pool = None


def _get_pool():
    global _pool
    if _pool is None:
        _pool = cf.ProcessPoolExecutor(max_workers=2)
    return _pool


def _verify(ground_truth: str, model_output: str) -> float:
    from .prime_math import compute_score as grade

    return float(grade(model_output, ground_truth)[0])


def compute_score(model_output: str, ground_truth: str, timeout_score: float = 0, timeout: float = 30.0) -> float:
    global _pool
    try:
        return _get_pool().submit(_verify, str(ground_truth), model_output).result(timeout=timeout)
    except cf.TimeoutError:
        if _pool is not None:
            _pool.shutdown(wait=False, cancel_futures=True)
            _pool = None
        return timeout_score
    except Exception:
        return 0.0
