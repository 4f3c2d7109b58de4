"""Code-contest grading: extract the last ```python block, run it against the input/output pairs of the test
cases in a child interpreter (resource limits, wall-clock timeout), return pass rate (``continuous``) or all-pass.

Parity target: ``verl/utils/reward_score/prime_code/{__init__ 73, utils 60, testing_util 696}.py``
(first a whole-suite run; if it fails and ``continuous``, the first 10 cases individually).
"""

from __future__ import annotations

import json

from .runner import run_cases

__all__ = ["compute_score", "extract_code"]


def extract_code(completion: str) -> str:
    return completion.split("```python")[-1].split("```")[0]


def compute_score(completion, test_cases, continuous: bool = False, timeout: float = 5.0):
    code = extract_code(completion)
    try:
        if not isinstance(test_cases, dict):
            test_cases = json.loads(test_cases)
        inputs, outputs = list(test_cases["inputs"]), list(test_cases["outputs"])
        fn_name = test_cases.get("fn_name")
    except Exception as e:  # malformed ground truth counts as a failure, not an exception in the trainer
        return False, [{"error": f"bad test_cases: {e}"}]
    res = run_cases(code, inputs, outputs, fn_name=fn_name, timeout=timeout)
    if all(r["passed"] for r in res):
        return True, res[:1]
    if not continuous:
        return False, res
    head = res[:10]
    return sum(r["passed"] for r in head) / max(1, len(head)), head
