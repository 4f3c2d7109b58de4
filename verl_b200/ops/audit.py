"""Audit mode for the index-driven operators: ``VERL_B200_AUDIT=1`` (or ``audit.enable()``).

The kernels trust the index tensors they are handed: token ids into the embedding table, positions into the rotary table,
slot numbers into the paged KV cache, block numbers in a block table, labels into the vocabulary. A wrong value there is the
usual way a correct kernel ends up reading or writing out of bounds, and on the device that shows up far from its cause, if
at all. In audit mode every such operator first checks its index tensors on the host side of the launch (one reduction and
a synchronising read per tensor: slow, so off by default) and raises ``AuditError`` naming the operator, the argument, the
first offending position and value and the allowed range. Nothing is launched for a call that fails. It also checks the
16-byte alignment the vectorised kernels assume. The checks are the same on CPU tensors, so they are tested without a GPU.
"""

from __future__ import annotations

import os
from contextlib import contextmanager
from typing import Optional

import torch

__all__ = ["AuditError", "enabled", "enable", "scope", "check_index", "check_aligned", "check_paged_cache"]

_ON = os.environ.get("VERL_B200_AUDIT", "0") == "1"


class AuditError(ValueError):
    pass


def enabled() -> bool:
    return _ON


def enable(on: bool = True) -> None:
    global _ON
    _ON = bool(on)


@contextmanager
def scope(on: bool = True):
    global _ON
    old, _ON = _ON, bool(on)
    try:
        yield
    finally:
        _ON = old


def _capturing(t: torch.Tensor) -> bool:
    """A check reads its verdict back to the host, which a stream that is being captured into a CUDA graph does not allow:
    the operators of a captured decode step are audited in the eager warm-up steps that precede the capture, not inside it."""
    return t.is_cuda and torch.cuda.is_current_stream_capturing()


def check_index(op: str, name: str, t: Optional[torch.Tensor], hi: int, lo: int = 0, skip_negative: bool = False) -> None:
    """Every element of ``t`` lies in ``[lo, hi)``; with ``skip_negative`` negative values mean "no entry" and pass."""
    if not _ON or t is None or t.numel() == 0 or _capturing(t):
        return
    if t.is_floating_point():
        raise AuditError(f"{op}: {name} must be an integer tensor, got {t.dtype}")
    flat = t.reshape(-1)
    bad = (flat >= hi) | (((flat >= 0) & (flat < lo)) if skip_negative else (flat < lo))
    n_bad = int(bad.sum())
    if n_bad:
        at = int(torch.nonzero(bad)[0])
        raise AuditError(f"{op}: {name} has {n_bad} value(s) outside [{lo}, {hi}); first at flat position {at}: {int(flat[at])} "
                         f"(shape {tuple(t.shape)})")


def check_aligned(op: str, name: str, t: Optional[torch.Tensor], nbytes: int = 16) -> None:
    if not _ON or t is None or t.numel() == 0:
        return
    if t.data_ptr() % nbytes:
        raise AuditError(f"{op}: {name} starts at an address that is not a multiple of {nbytes} bytes (offset {t.data_ptr() % nbytes})")
    if t.dim() >= 2 and t.stride(-1) == 1 and (t.stride(-2) * t.element_size()) % nbytes:
        raise AuditError(f"{op}: rows of {name} are {t.stride(-2) * t.element_size()} bytes apart, not a multiple of {nbytes}")


def check_paged_cache(op: str, block_table: torch.Tensor, ctx_len: torch.Tensor, num_blocks: int, block_size: int) -> None:
    """Block numbers that a sequence's context actually reaches are valid blocks, and the context fits its table row."""
    if not _ON or block_table.numel() == 0 or _capturing(block_table):
        return
    max_ctx = block_table.shape[1] * block_size
    check_index(op, "ctx_len", ctx_len, max_ctx + 1)
    used = (torch.arange(block_table.shape[1], device=block_table.device)[None, :] * block_size) < ctx_len.reshape(-1, 1)
    vals = torch.where(used, block_table, torch.zeros_like(block_table))
    check_index(op, "block_table (entries within each sequence's context)", vals, num_blocks)
