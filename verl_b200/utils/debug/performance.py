"""Kept for code that imports the timing helpers from their old place; they live in ``utils/profiler/performance.py``.
Parity target: ``verl/utils/debug/performance.py``."""

from ..profiler.performance import reduce_timing, simple_timer  # noqa: F401

__all__ = ["reduce_timing", "simple_timer"]
