"""Loader of the in-tree sm_100a library and thin typed wrappers over ``torch.ops.verl_b200``.

On a machine with a CUDA device the native library is mandatory: a missing or unbuildable library
raises instead of silently falling back to PyTorch kernels.
"""

from __future__ import annotations

import ctypes
import threading

import torch

from . import build as _build

_lock = threading.Lock()
_loaded = False
_cdll = None


def lib_path():
    return _build.LIB


def load(build_if_missing: bool = True) -> bool:
    """Load ``_C.so`` into the process (idempotent). Returns True when the ops are registered."""
    global _loaded
    if _loaded:
        return True
    with _lock:
        if _loaded:
            return True
        if not _build.LIB.exists() or not _build.is_current():
            if not build_if_missing:
                return False
            _build.build()
        torch.ops.load_library(str(_build.LIB))
        _loaded = True
    return True


def cdll() -> ctypes.CDLL:
    """ctypes handle on the same shared object (for the exported C entry points)."""
    global _cdll
    load()
    if _cdll is None:
        _cdll = ctypes.CDLL(str(_build.LIB))
    return _cdll


def available() -> bool:
    """True when a CUDA device is present (native kernels are then required, not optional)."""
    return torch.cuda.is_available()


def ops():
    load()
    return torch.ops.verl_b200


def check_status() -> None:
    """Raise if any kernel recorded a timed-out wait since the last check (synchronises the device)."""
    code = int(ops().gemm_status())
    if code != 0:
        raise RuntimeError(f"verl_b200 native kernel reported status {code} (a bounded in-kernel wait ran out)")


def launch_count() -> int:
    """Kernels of this library launched so far by this process (graph replays are added by their owners)."""
    return int(ops().launch_count()) if _loaded or available() else 0


def add_launches(n: int) -> None:
    ops().add_launches(int(n))
