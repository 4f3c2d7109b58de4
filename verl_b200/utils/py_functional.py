"""Small Python helpers used across the framework: a portable time limit for function calls, dictionary utilities for
metric accumulation, an enum whose members are registered at run time, scoped environment variables.

Parity target: ``verl/utils/py_functional.py`` (``timeout_limit`` :56, ``union_two_dict`` :151, ``rename_dict`` :169,
``append_to_dict`` :187, ``NestedNamespace`` :210, ``DynamicEnum`` :259, ``temp_env_var`` :303,
``convert_to_regular_types`` :333, ``list_of_dict_to_dict_of_list`` :359).
"""

from __future__ import annotations

import contextlib
import functools
import multiprocessing
import os
import signal
import threading
from types import SimpleNamespace
from typing import Any, Callable, Iterator, Optional

__all__ = ["timeout_limit", "union_two_dict", "rename_dict", "append_to_dict", "NestedNamespace", "DynamicEnum",
           "temp_env_var", "convert_to_regular_types", "convert_nested_value_to_list_recursive", "list_of_dict_to_dict_of_list"]


def _child(fn: Callable, q, args: tuple, kwargs: dict) -> None:
    try:
        q.put((True, fn(*args, **kwargs)))
    except BaseException as e:  # the parent re-raises
        q.put((False, e))


def timeout_limit(seconds: float, use_signals: bool = False):
    """Decorator: the call raises ``TimeoutError`` after ``seconds``. With ``use_signals`` (main thread, POSIX) the call
    runs in place under ``SIGALRM``; otherwise it runs in a child process that is terminated on expiry, which also works
    from worker threads and for code that never returns to the interpreter."""

    def decorator(fn: Callable):
        @functools.wraps(fn)
        def with_signal(*args, **kwargs):
            def on_alarm(signum, frame):
                raise TimeoutError(f"{fn.__name__} exceeded {seconds} s")

            old = signal.signal(signal.SIGALRM, on_alarm)
            signal.setitimer(signal.ITIMER_REAL, seconds)
            try:
                return fn(*args, **kwargs)
            finally:
                signal.setitimer(signal.ITIMER_REAL, 0)
                signal.signal(signal.SIGALRM, old)

        @functools.wraps(fn)
        def with_process(*args, **kwargs):
            ctx = multiprocessing.get_context("fork" if hasattr(os, "fork") else "spawn")
            q = ctx.Queue(1)
            p = ctx.Process(target=_child, args=(fn, q, args, kwargs))
            p.start()
            p.join(seconds)
            if p.is_alive():
                p.terminate()
                p.join(1.0)
                if p.is_alive():
                    p.kill()
                    p.join()
                raise TimeoutError(f"{fn.__name__} exceeded {seconds} s")
            if q.empty():
                raise RuntimeError(f"{fn.__name__}: the child exited with code {p.exitcode} without a result")
            ok, val = q.get()
            if not ok:
                raise val
            return val

        if use_signals and threading.current_thread() is threading.main_thread() and hasattr(signal, "SIGALRM"):
            return with_signal
        return with_process

    return decorator


def union_two_dict(dict1: dict, dict2: dict) -> dict:
    """In-place union; a key present in both must carry the same value."""
    for k, v in dict2.items():
        if k in dict1:
            assert dict1[k] == v, f"{k}: conflicting values {dict1[k]!r} and {v!r}"
        dict1[k] = v
    return dict1


def rename_dict(data: dict, prefix: str = "") -> dict:
    return {f"{prefix}{k}": v for k, v in data.items()}


def append_to_dict(data: dict, new_data: dict, prefix: str = "") -> None:
    """``data[prefix + key]`` is a list that collects the values seen so far (list values are extended, not nested)."""
    for k, v in new_data.items():
        dst = data.setdefault(f"{prefix}{k}", [])
        if isinstance(v, list):
            dst.extend(v)
        else:
            dst.append(v)


class NestedNamespace(SimpleNamespace):
    """Attribute access to a nested dictionary (dictionaries inside lists included)."""

    def __init__(self, dictionary: dict, **kwargs):
        super().__init__(**kwargs)
        for k, v in dictionary.items():
            setattr(self, k, self._wrap(v))

    @classmethod
    def _wrap(cls, v):
        if isinstance(v, dict):
            return cls(v)
        if isinstance(v, list):
            return [cls._wrap(x) for x in v]
        return v


class _DynamicEnumMeta(type):
    def __iter__(cls) -> Iterator[Any]:
        return iter(cls._registry.values())

    def __contains__(cls, item: Any) -> bool:
        return item in cls._registry or item in cls._registry.values()

    def __getitem__(cls, name: str) -> Any:
        return cls._registry[name]

    def names(cls):
        return list(cls._registry.keys())

    def values(cls):
        return list(cls._registry.values())


class DynamicEnum(metaclass=_DynamicEnumMeta):
    """Enum-like class whose members are added with ``register`` at run time; each subclass sets its own ``_registry``
    and ``_next_value``. Members pickle by name."""

    _registry: dict = {}
    _next_value: int = 0

    def __init__(self, name: str, value: int):
        self.name, self.value = name, value

    def __repr__(self) -> str:
        return f"<{type(self).__name__}.{self.name}: {self.value}>"

    def __reduce_ex__(self, protocol):
        return getattr, (type(self), self.name)

    @classmethod
    def register(cls, name: str) -> "DynamicEnum":
        key = name.upper()
        if key in cls._registry:
            raise ValueError(f"{key} is already a member of {cls.__name__}")
        member = cls(key, cls._next_value)
        cls._registry[key] = member
        setattr(cls, key, member)
        cls._next_value += 1
        return member

    @classmethod
    def remove(cls, name: str) -> "DynamicEnum":
        key = name.upper()
        member = cls._registry.pop(key)
        delattr(cls, key)
        return member

    @classmethod
    def from_name(cls, name: str) -> Optional["DynamicEnum"]:
        return cls._registry.get(name.upper())


@contextlib.contextmanager
def temp_env_var(key: str, value: str):
    old = os.environ.get(key)
    os.environ[key] = value
    try:
        yield
    finally:
        if old is None:
            os.environ.pop(key, None)
        else:
            os.environ[key] = old


def convert_to_regular_types(obj):
    """Config containers (anything with ``items`` / list-likes) -> plain dicts and lists, recursively."""
    if hasattr(obj, "items") and not isinstance(obj, dict):
        obj = dict(obj.items())
    if isinstance(obj, dict):
        return {k: convert_to_regular_types(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)) or (hasattr(obj, "__iter__") and hasattr(obj, "__len__") and not isinstance(obj, (str, bytes))
                                          and type(obj).__name__ in ("ListConfig", "ConfigList")):
        return [convert_to_regular_types(v) for v in obj]
    return obj


def convert_nested_value_to_list_recursive(data_item):
    """numpy arrays / tensors anywhere inside nested dicts and lists become lists (JSON-friendly)."""
    if isinstance(data_item, dict):
        return {k: convert_nested_value_to_list_recursive(v) for k, v in data_item.items()}
    if isinstance(data_item, (list, tuple)):
        return [convert_nested_value_to_list_recursive(v) for v in data_item]
    if hasattr(data_item, "tolist"):
        return convert_nested_value_to_list_recursive(data_item.tolist())
    return data_item


def list_of_dict_to_dict_of_list(list_of_dict: list[dict]) -> dict:
    if not list_of_dict:
        return {}
    keys = list_of_dict[0].keys()
    out = {k: [] for k in keys}
    for d in list_of_dict:
        assert d.keys() == keys, "all dictionaries must have the same keys"
        for k, v in d.items():
            out[k].append(v)
    return out
