"""Rule rewards: math normalisation/grading, code execution in a limited child process, QA exact match, dispatch."""
import json

from verl_b200.utils.reward_score import default_compute_score, geo3k, prime_code, prime_math
from verl_b200.utils.reward_score import search_r1_like_qa_em as qa


def test_prime_math_equivalences():
    ok = lambda out, gt: prime_math.compute_score(out, gt)[0]
    assert ok("so \\boxed{\\frac{1}{2}}", "0.5") and ok("\\boxed{(1, 2.0)}", "(1,2)") and ok("the answer is 1,234 meters.", "1234")
    assert ok("\\boxed{50\\%}", "50") and ok("\\boxed{\\dfrac{3}{4}}", "\\frac{3}{4}")
    assert not ok("\\boxed{3}", "4") and not ok("no answer here", "4")
    assert not ok("\\boxed{[1,2)}", "(1,2)")


def test_prime_code_stdin_call_based_timeouts_and_crashes():
    cases = {"inputs": ["2\n", "5\n"], "outputs": ["4\n", "10\n"]}
    assert prime_code.compute_score("```python\nn=int(input())\nprint(n*2)\n```", cases, continuous=True)[0] is True
    assert prime_code.compute_score("```python\nn=int(input())\nprint(n*2 if n<3 else 0)\n```", json.dumps(cases), continuous=True)[0] == 0.5
    assert prime_code.compute_score("while True: pass", cases, continuous=True, timeout=1.0)[0] == 0.0
    assert prime_code.compute_score("raise SystemExit(3)", cases)[0] is False
    call = {"fn_name": "add", "inputs": [[1, 2], [3, 4]], "outputs": [[3], [7]]}
    assert prime_code.compute_score("class Solution:\n    def add(self, a, b):\n        return a + b", call)[0] is True


def test_geo3k_and_qa_and_dispatch():
    assert geo3k.compute_score("<think>x</think> so \\boxed{12}", "12") == 1.0
    assert abs(geo3k.compute_score("\\boxed{12}", "12") - 0.9) < 1e-9
    assert qa.compute_score("<answer>The Eiffel Tower.</answer>", {"target": ["eiffel tower"]}) == 1.0
    assert qa.compute_score("<answer>a</answer>" * 11 + "<answer>eiffel tower</answer>", {"target": ["eiffel tower"]}) == 0.25
    assert qa.compute_score("nothing", {"target": ["x"]}) == 0
    assert qa.compute_score_subem("<answer>it is the eiffel tower in paris</answer>", {"target": "Eiffel Tower"}) == 1.0
    assert default_compute_score("numina_olympiads", "\\boxed{7}", "7") == 1.0
    assert default_compute_score("nq", "<answer>x</answer>", {"target": ["x"]}) == 1.0
    assert default_compute_score("hiyouga/geometry3k", "<think>a</think>\\boxed{1}", "1") == 1.0
    assert default_compute_score("apps", "print(input())", {"inputs": ["a\n"], "outputs": ["a\n"]}) == 1.0


def test_sandbox_client_against_local_stub():
    import http.server
    import threading

    from verl_b200.utils.reward_score import sandbox_fusion

    class H(http.server.BaseHTTPRequestHandler):
        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            out = str(int(body["stdin"]) * 2) if "n*2" in body["code"] else "?"
            data = json.dumps({"status": "Success", "run_result": {"return_code": 0, "stdout": out, "stderr": ""}}).encode()
            self.send_response(200)
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def log_message(self, *a):
            pass

    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    url = f"http://127.0.0.1:{srv.server_address[1]}/run_code"
    cases = {"inputs": ["2", "5"], "outputs": ["4", "10"]}
    sem = threading.Semaphore(2)
    assert sandbox_fusion.compute_score(url, sem, 512, "```python\nprint(n*2)\n```", cases)[0] == 1.0
    assert sandbox_fusion.compute_score(url, sem, 512, "print(1)", cases, continuous=True)[0] == 0.0
    srv.shutdown()
