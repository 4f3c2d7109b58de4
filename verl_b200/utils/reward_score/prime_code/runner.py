"""Runs untrusted candidate programs in a separate interpreter with CPU/memory/file limits.

Two modes, as in the contest datasets: *stdin* programs (the input is fed on standard input, standard output is
compared token-wise with float tolerance) and *call-based* problems (``fn_name`` given: the function — or a method of
``Solution`` — is called with the JSON-decoded arguments and the return value compared).
"""

from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile

_PRELUDE = """
import sys, json
sys.setrecursionlimit(1 << 16)
def _limits():
    try:
        import resource
        resource.setrlimit(resource.RLIMIT_AS, ({mem}, {mem}))
        resource.setrlimit(resource.RLIMIT_CPU, ({cpu}, {cpu}))
        resource.setrlimit(resource.RLIMIT_FSIZE, (1 << 20, 1 << 20))
        resource.setrlimit(resource.RLIMIT_NPROC, (0, 0))
    except Exception:
        pass
_limits()
"""

_CALL_DRIVER = """
_args = json.loads(sys.stdin.read())
_ns = globals()
if "Solution" in _ns and hasattr(_ns["Solution"], {fn!r}):
    _res = getattr(_ns["Solution"](), {fn!r})(*_args)
else:
    _res = _ns[{fn!r}](*_args)
if isinstance(_res, tuple):
    _res = list(_res)
print("\\n__RESULT__" + json.dumps(_res))
"""


def _same_tokens(a: str, b: str) -> bool:
    ta, tb = a.split(), b.split()
    if len(ta) != len(tb):
        return False
    for x, y in zip(ta, tb):
        if x == y:
            continue
        try:
            if abs(float(x) - float(y)) > 1e-6 * max(1.0, abs(float(y))):
                return False
        except ValueError:
            return False
    return True


def _run(path: str, stdin: str, timeout: float):
    env = {"PATH": os.environ.get("PATH", ""), "PYTHONHASHSEED": "0"}
    try:
        p = subprocess.run([sys.executable, "-I", path], input=stdin, capture_output=True, text=True, timeout=timeout,
                           env=env, cwd=os.path.dirname(path))
        return p.returncode, p.stdout, p.stderr[-500:]
    except subprocess.TimeoutExpired:
        return -9, "", "timeout"


def run_cases(code: str, inputs: list, outputs: list, fn_name=None, timeout: float = 5.0, memory_mb: int = 1024) -> list[dict]:
    src = _PRELUDE.format(mem=memory_mb << 20, cpu=int(timeout) + 1) + "\n" + code + "\n"
    if fn_name:
        src += _CALL_DRIVER.format(fn=fn_name)
    results = []
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "candidate.py")
        with open(path, "w") as f:
            f.write(src)
        for inp, want in zip(inputs, outputs):
            if fn_name:
                rc, out, err = _run(path, json.dumps(inp), timeout)
                ok = False
                if rc == 0 and "__RESULT__" in out:
                    try:
                        got = json.loads(out.rsplit("__RESULT__", 1)[1])
                        exp = want[0] if isinstance(want, list) and len(want) == 1 and not isinstance(got, list) else want
                        ok = got == exp or (isinstance(want, list) and len(want) == 1 and got == want[0])
                    except Exception:
                        ok = False
            else:
                text_in = inp if isinstance(inp, str) else "\n".join(map(str, inp))
                text_out = want if isinstance(want, str) else "\n".join(map(str, want))
                rc, out, err = _run(path, text_in, timeout)
                ok = rc == 0 and _same_tokens(out, text_out)
            results.append({"passed": bool(ok), "returncode": rc, "stderr": err if not ok else ""})
    return results
