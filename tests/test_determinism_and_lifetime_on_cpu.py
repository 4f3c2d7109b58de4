"""Run-twice bitwise determinism of a training step, and workers that die with their parent."""
import os
import signal
import subprocess
import sys
import time
from functools import partial

import torch

os.environ["VERL_ENGINE_DEVICE"] = "cpu"


def _two_steps(preset: str):
    from verl_b200.models import get_preset
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
    from verl_b200.workers.engine.utils import enable_full_determinism
    from verl_b200.workers.utils.losses import sft_loss

    enable_full_determinism(11)
    eng = NativeEngineWithLMHead(get_preset(preset), FSDPEngineConfig(seed=3, micro_batch_size_per_gpu=2), OptimizerConfig(lr=1e-2))
    eng.initialize()
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(3, 500, (4, 20), generator=g)
    am = torch.ones_like(ids)
    data = {"input_ids": ids, "attention_mask": am, "responses": ids[:, -8:], "response_mask": am[:, -8:]}
    norms = [eng.train_batch(dict(data), partial(sft_loss, None))["metrics"]["grad_norm"] for _ in range(2)]
    return norms, eng.params.flat.clone()


def test_training_step_is_bitwise_reproducible():
    for preset in ("tiny-llama", "tiny-moe"):
        n1, w1 = _two_steps(preset)
        n2, w2 = _two_steps(preset)
        assert n1 == n2 and torch.equal(w1, w2), preset
    torch.use_deterministic_algorithms(False)
    from verl_b200.ops import functional as F

    F.DETERMINISTIC_ATTENTION = False


CHILD = r"""
import os, sys, time, multiprocessing as mp
sys.path.insert(0, {repo!r})
from verl_b200.utils.process import set_death_signal

def grandchild(path):
    assert set_death_signal()
    open(path, "w").write(str(os.getpid()))
    time.sleep(120)

if __name__ == "__main__":
    p = mp.get_context("fork").Process(target=grandchild, args=(sys.argv[1],))
    p.start()
    time.sleep(120)
"""


def test_worker_dies_with_its_parent(tmp_path):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "child.py"
    script.write_text(CHILD.format(repo=repo))
    pidfile = tmp_path / "pid"
    child = subprocess.Popen([sys.executable, str(script), str(pidfile)])
    try:
        for _ in range(200):
            if pidfile.exists() and pidfile.read_text():
                break
            time.sleep(0.05)
        gpid = int(pidfile.read_text())
        os.kill(gpid, 0)                      # the grandchild is alive
        child.send_signal(signal.SIGKILL)     # the parent dies without any clean-up
        child.wait(timeout=10)
        for _ in range(100):
            try:
                os.kill(gpid, 0)
            except ProcessLookupError:
                break
            time.sleep(0.05)
        else:
            os.kill(gpid, signal.SIGKILL)
            raise AssertionError("the grandchild outlived its parent")
    finally:
        if child.poll() is None:
            child.kill()
