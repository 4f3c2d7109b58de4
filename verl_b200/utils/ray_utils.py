"""Helpers around Ray and asyncio that the single-controller code uses when the Ray back-end is active. Ray itself is
imported lazily: everything except ``parallel_put`` works without it.

Parity target: ``verl/utils/ray_utils.py`` (``ray_noset_visible_devices`` :28, ``parallel_put`` :51, ``get_event_loop``
:87, ``auto_await`` :97).
"""

from __future__ import annotations

import asyncio
import concurrent.futures
import functools
import inspect
import os
from typing import Any, Optional

__all__ = ["ray_noset_visible_devices", "parallel_put", "get_event_loop", "auto_await"]

_NOSET_VARS = ("RAY_EXPERIMENTAL_NOSET_CUDA_VISIBLE_DEVICES", "RAY_EXPERIMENTAL_NOSET_ROCR_VISIBLE_DEVICES",
               "RAY_EXPERIMENTAL_NOSET_HIP_VISIBLE_DEVICES", "RAY_EXPERIMENTAL_NOSET_ASCEND_RT_VISIBLE_DEVICES")


def ray_noset_visible_devices(env_vars=os.environ) -> bool:
    """True when Ray was told not to rewrite the device-visibility variables: workers then pick their device by local
    rank instead of assuming device 0."""
    return any(env_vars.get(k) for k in _NOSET_VARS)


def parallel_put(data_list: list[Any], max_workers: Optional[int] = None) -> list:
    """``ray.put`` of many objects from a thread pool; results keep the input order."""
    import ray

    if not data_list:
        return []
    workers = max_workers or min(len(data_list), 16)
    with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
        return list(pool.map(ray.put, data_list))


def get_event_loop() -> asyncio.AbstractEventLoop:
    try:
        return asyncio.get_event_loop()
    except RuntimeError:
        loop = asyncio.new_event_loop()
        asyncio.set_event_loop(loop)
        return loop


def auto_await(func):
    """A coroutine function that can also be called from synchronous code: outside a running loop the call blocks until
    the coroutine finishes, inside one it returns the awaitable."""
    if not inspect.iscoroutinefunction(func):
        return func

    @functools.wraps(func)
    def wrapper(*args, **kwargs):
        coro = func(*args, **kwargs)
        try:
            asyncio.get_running_loop()
        except RuntimeError:
            return asyncio.run(coro)
        return coro

    return wrapper
