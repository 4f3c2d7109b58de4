"""Remote code-execution grading through a SandboxFusion-style HTTP service (``POST <url>`` with code, stdin and
limits; JSON verdict back), with a bounded number of concurrent requests.

Parity target: ``verl/utils/reward_score/sandbox_fusion/{__init__ 121, utils 578}.py``. There is no network in
this build's test environment: the client is exercised against a local stub server.
"""

from __future__ import annotations

import concurrent.futures as cf
import json
import threading
from typing import Optional

__all__ = ["compute_score", "call_sandbox_api", "check_correctness"]


def call_sandbox_api(url: str, code: str, stdin: str, compile_timeout=10, run_timeout=10, memory_limit_mb=1024,
                     language="python", retries: int = 3):
    import requests

    payload = {"code": code, "stdin": stdin, "compile_timeout": compile_timeout, "run_timeout": run_timeout,
               "memory_limit_MB": memory_limit_mb, "language": language}
    last = None
    for _ in range(retries):
        try:
            r = requests.post(url, json=payload, timeout=compile_timeout + run_timeout + 10)
            if r.status_code == 200:
                return r.json(), None
            last = f"HTTP {r.status_code}"
            if r.status_code < 500 and r.status_code != 429:
                break
        except Exception as e:  # connection errors are retried
            last = repr(e)
    return None, last


def _tokens_equal(a: str, b: str) -> bool:
    return a.split() == b.split()


def check_correctness(url, in_outs: dict, code: str, timeout=10, memory_limit_mb=1024, language="python",
                      semaphore: Optional[threading.Semaphore] = None, max_workers: int = 8):
    inputs, outputs = in_outs.get("inputs", []), in_outs.get("outputs", [])

    def one(i):
        if semaphore is not None:
            semaphore.acquire()
        try:
            resp, err = call_sandbox_api(url, code, str(inputs[i]), run_timeout=timeout, memory_limit_mb=memory_limit_mb,
                                         language=language)
        finally:
            if semaphore is not None:
                semaphore.release()
        if resp is None:
            return -1, {"api_error": err}
        run = resp.get("run_result") or {}
        if resp.get("status") != "Success" or run.get("return_code", 1) != 0:
            return False, {"status": resp.get("status"), "stderr": str(run.get("stderr", ""))[-300:]}
        return _tokens_equal(str(run.get("stdout", "")), str(outputs[i])), {}

    with cf.ThreadPoolExecutor(max_workers=max(1, min(max_workers, len(inputs) or 1))) as ex:
        res = list(ex.map(one, range(len(inputs))))
    return [r[0] for r in res], [r[1] for r in res]


def compute_score(sandbox_fusion_url, concurrent_semaphore, memory_limit_mb, completion, test_cases, continuous=False,
                  timeout=10):
    code = completion.split("```python")[-1].split("```")[0] if "```python" in completion else completion
    if not isinstance(test_cases, dict):
        try:
            test_cases = json.loads(test_cases)
        except Exception as e:
            return 0.0, [{"error": f"bad test_cases: {e}"}]
    res, meta = check_correctness(sandbox_fusion_url, test_cases, code, timeout=timeout,
                                  memory_limit_mb=memory_limit_mb or 1024, semaphore=concurrent_semaphore)
    if not res:
        return 0.0, meta
    passed = sum(1 for r in res if r is True)
    return (passed / len(res) if continuous else float(passed == len(res))), meta
