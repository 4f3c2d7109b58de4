"""Process-lifetime helpers: children that must not outlive their parent.

Parity target: ``verl/workers/rollout/vllm_rollout/utils.py:71`` (``set_death_signal``: workers die with the process that
spawned them, so a crashed controller leaves no orphans holding GPUs).
"""

from __future__ import annotations

import ctypes
import os
import signal
import sys

__all__ = ["set_death_signal"]

_PR_SET_PDEATHSIG = 1


def set_death_signal(sig: int = signal.SIGKILL) -> bool:
    """Ask the kernel to deliver ``sig`` to this process when its parent exits (Linux ``prctl(PR_SET_PDEATHSIG)``).
    Returns False where that is not available. If the parent is already gone the process exits at once."""
    if not sys.platform.startswith("linux"):
        return False
    parent = os.getppid()
    try:
        libc = ctypes.CDLL("libc.so.6", use_errno=True)
        if libc.prctl(_PR_SET_PDEATHSIG, int(sig), 0, 0, 0) != 0:
            return False
    except OSError:
        return False
    if os.getppid() != parent:  # the parent died between fork and prctl
        os.kill(os.getpid(), sig)
    return True
