"""Resource pools and the driver-side worker-group proxy.

Parity target: ``verl/single_controller/base/worker_group.py`` (``ResourcePool`` :27, ``ClassWithInitArgs`` :76,
aliveness check :102-183, ``_bind_worker_method`` :185-255).
"""

from __future__ import annotations

import logging
import signal
import threading
import time
from typing import Any, Callable

from .decorator import MAGIC_ATTR, Dispatch, get_predefined_dispatch_fn, get_predefined_execute_fn

__all__ = ["ResourcePool", "ClassWithInitArgs", "WorkerGroup", "check_workers_alive"]


class ResourcePool:
    """``process_on_nodes[i]`` worker processes on node ``i``; ``max_colocate_count`` roles may share a device."""

    def __init__(self, process_on_nodes=None, max_colocate_count: int = 10, n_gpus_per_node: int = 8) -> None:
        self._store = list(process_on_nodes or [])
        self.max_colocate_count = max_colocate_count
        self.n_gpus_per_node = n_gpus_per_node

    def add_node(self, process_count: int) -> None:
        self._store.append(process_count)

    @property
    def world_size(self) -> int:
        return sum(self._store)

    def __call__(self) -> Any:
        return self._store

    @property
    def store(self):
        return self._store

    def local_world_size_list(self) -> list[int]:
        return [n for n in self._store for _ in range(n)]

    def local_rank_list(self) -> list[int]:
        return [i for n in self._store for i in range(n)]


class ClassWithInitArgs:
    """A class plus the arguments to construct it with, so instantiation can happen on the worker side."""

    def __init__(self, cls, *args, **kwargs) -> None:
        self.cls, self.args, self.kwargs = cls, args, kwargs
        self.fused_worker_used = False

    def __call__(self) -> Any:
        return self.cls(*self.args, **self.kwargs)


def check_workers_alive(workers: list, is_alive: Callable, gap_time: float = 1) -> None:
    """Poll worker liveness; a dead worker raises SIGABRT in the main thread of the driver."""
    while True:
        for w in workers:
            if not is_alive(w):
                logging.warning(f"worker {w} is not alive; sending SIGABRT to the main thread")
                signal.raise_signal(signal.SIGABRT)
        time.sleep(gap_time)


class WorkerGroup:
    fused_worker_execute_fn_name = "_fuw_execute"

    def __init__(self, resource_pool: ResourcePool | None = None, **kwargs) -> None:
        self._is_init_with_detached_workers = resource_pool is None
        self.fused_worker_used = False
        self._procecss_dispatch_config = resource_pool() if resource_pool is not None else None
        self._workers: list = []
        self._worker_names: list = []
        self._dispatch_info: dict = {}
        self._collect_info: dict = {}
        self._master_addr = None
        self._master_port = None
        self._checker_thread = None

    def _is_worker_alive(self, worker) -> bool:
        raise NotImplementedError("WorkerGroup._is_worker_alive called, should be implemented in derived class.")

    def _block_until_all_workers_alive(self) -> None:
        while not all(self._is_worker_alive(w) for w in self._workers):
            time.sleep(1)

    def start_worker_aliveness_check(self, every_n_seconds: float = 1) -> None:
        self._block_until_all_workers_alive()
        self._checker_thread = threading.Thread(target=check_workers_alive, daemon=True,
                                                args=(self._workers, self._is_worker_alive, every_n_seconds))
        self._checker_thread.start()

    @property
    def world_size(self) -> int:
        return len(self._workers)

    # -- lazy dispatch-mesh queries (overridable by backends)
    def _query_dispatch_info(self, mesh_name: str) -> list[int]:
        return self.execute_all_sync("_query_dispatch_info", mesh_name)

    def _query_collect_info(self, mesh_name: str) -> list[bool]:
        return self.execute_all_sync("_query_collect_info", mesh_name)

    def _bind_worker_method(self, user_defined_cls, func_generator) -> list[str]:
        """Create a proxy method on ``self`` for every ``@register``-ed method of ``user_defined_cls``."""
        bound = []
        for name in dir(user_defined_cls):
            try:
                method = getattr(user_defined_cls, name)
                assert callable(method)
            except Exception:
                continue
            if not hasattr(method, MAGIC_ATTR):
                continue
            attrs = getattr(method, MAGIC_ATTR)
            mode = attrs["dispatch_mode"]
            fns = get_predefined_dispatch_fn(mode) if isinstance(mode, Dispatch) else mode
            exec_name = get_predefined_execute_fn(attrs["execute_mode"])["execute_fn_name"]
            try:
                execute_fn = getattr(self, exec_name)
            except AttributeError:
                raise AttributeError(f"execute_fn {exec_name} is not defined on {type(self).__name__}") from None
            proxy = func_generator(self, name, dispatch_fn=fns["dispatch_fn"], collect_fn=fns["collect_fn"],
                                   execute_fn=execute_fn, blocking=attrs["blocking"])
            setattr(self, name, proxy)
            bound.append(name)
        return bound
