"""Span tracing of agent-loop trajectories (weave / mlflow / trackio when installed; otherwise an in-memory
ring that tests and debuggers can read). Parity target: ``verl/utils/rollout_trace.py`` (471 lines)."""

from __future__ import annotations

import contextlib
import contextvars
import functools
import inspect
import time
from collections import deque
from typing import Optional

__all__ = ["RolloutTraceConfig", "rollout_trace_op", "rollout_trace_attr", "TRACE_RING"]

TRACE_RING: deque = deque(maxlen=4096)


class RolloutTraceConfig:
    _instance = None
    backend: Optional[str] = None
    token2text: bool = False
    project_name: str = ""
    experiment_name: str = ""
    max_samples_per_step_per_worker: Optional[int] = None

    @classmethod
    def get_instance(cls):
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    @classmethod
    def init(cls, project_name: str, experiment_name: str, backend: Optional[str], token2text: bool = False,
             max_samples_per_step_per_worker: Optional[int] = None):
        c = cls.get_instance()
        c.project_name, c.experiment_name, c.backend, c.token2text = project_name, experiment_name, backend, token2text
        c.max_samples_per_step_per_worker = max_samples_per_step_per_worker
        if backend == "weave":
            import weave

            weave.init(project_name)
        elif backend == "mlflow":
            import mlflow

            mlflow.set_experiment(project_name)
        elif backend not in (None, "memory", "trackio"):
            raise ValueError(f"Unknown rollout trace backend: {backend}")

    @classmethod
    def get_backend(cls):
        return cls.get_instance().backend

    @classmethod
    def reset(cls):
        cls._instance = None


# Attributes of the trajectory that the current task works on. A context variable, not a global stack: the trajectories
# of a batch run as concurrent asyncio tasks, each of which sees only the attributes it set itself.
_trace_attrs: contextvars.ContextVar = contextvars.ContextVar("rollout_trace_attrs", default=None)


@contextlib.contextmanager
def rollout_trace_attr(sample_index=None, step=None, rollout_n=None, name="rollout_trace", validate=False, trace: bool = True):
    """Spans recorded inside carry these attributes; ``trace=False`` records none (a sampled-out trajectory)."""
    token = _trace_attrs.set({"sample_index": sample_index, "step": step, "rollout_n": rollout_n, "validate": validate,
                              "_trace": bool(trace)})
    try:
        yield
    finally:
        _trace_attrs.reset(token)


def rollout_trace_op(fn):
    """Record a span (name, duration, attributes) around an (async) method when tracing is enabled."""

    def record(name, t0, ok):
        if RolloutTraceConfig.get_backend() is not None:
            attrs = dict(_trace_attrs.get() or {})
            if attrs.pop("_trace", True):
                TRACE_RING.append({"op": name, "seconds": time.time() - t0, "ok": ok, **attrs})

    if inspect.iscoroutinefunction(fn):
        @functools.wraps(fn)
        async def aw(*a, **k):
            t0 = time.time()
            try:
                out = await fn(*a, **k)
                record(fn.__qualname__, t0, True)
                return out
            except Exception:
                record(fn.__qualname__, t0, False)
                raise

        return aw

    @functools.wraps(fn)
    def w(*a, **k):
        t0 = time.time()
        try:
            out = fn(*a, **k)
            record(fn.__qualname__, t0, True)
            return out
        except Exception:
            record(fn.__qualname__, t0, False)
            raise

    return w
