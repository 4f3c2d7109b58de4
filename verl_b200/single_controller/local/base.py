"""Ray-free worker-group backends.

* :class:`InProcessWorkerGroup` — N worker instances inside the driver process (a fake cluster for dispatch
  semantics and CPU unit tests; the role Ray CPU actors play in the reference's tests).
* :class:`MultiprocessWorkerGroup` — one OS process per rank (one per GPU), driven over pipes by the single
  controller; ranks rendezvous through ``MASTER_ADDR/MASTER_PORT`` (gloo on CPU, NCCL on GPU).
* :class:`SPMDWorkerGroup` — for ``torchrun`` launches: every rank runs the controller program on its own
  shard of the batch, so dispatch and collect are the identity and data never leaves the GPU it lives on.

Reference behaviour studied: ``verl/single_controller/ray/base.py`` (``func_generator`` :49-67, ``RayWorkerGroup``
:418-890) — re-designed without an object store.
"""

from __future__ import annotations

import multiprocessing as mp
import os
import socket
import traceback
from concurrent.futures import Future
from typing import Any, Optional

from ...protocol import DataProto, DataProtoConfig, DataProtoFuture, unpad_dataproto
from ..base.worker_group import ClassWithInitArgs, ResourcePool, WorkerGroup

__all__ = ["InProcessWorkerGroup", "MultiprocessWorkerGroup", "SPMDWorkerGroup", "func_generator"]


def _resolve(x):
    if isinstance(x, Future):
        return x.result()
    if isinstance(x, list):
        return [_resolve(v) for v in x]
    return x


def func_generator(self, method_name, dispatch_fn, collect_fn, execute_fn, blocking):
    class Functor:
        def __call__(this, *args, **kwargs):
            args, kwargs = dispatch_fn(self, *args, **kwargs)
            pad = kwargs.pop(DataProtoConfig.auto_padding_key, None)
            output = execute_fn(method_name, *args, **kwargs)
            if blocking:
                output = _resolve(output)
            output = collect_fn(self, output)
            if pad and isinstance(output, DataProto):
                output = unpad_dataproto(output, pad[0] if isinstance(pad, list) else pad)
            return output

    return type(method_name, (Functor,), {})()


class _LocalGroupBase(WorkerGroup):
    def __init__(self, resource_pool=None, cls_with_init: Optional[ClassWithInitArgs] = None, **kwargs):
        super().__init__(resource_pool=resource_pool, **kwargs)
        self.cls_with_init = cls_with_init

    def _bind(self):
        self._bind_worker_method(self.cls_with_init.cls, func_generator)

    # -- execution primitives the proxies use
    def execute_all(self, method_name: str, *args, **kwargs):
        return self.execute_all_async(method_name, *args, **kwargs)

    def execute_all_sync(self, method_name: str, *args, **kwargs):
        return _resolve(self.execute_all_async(method_name, *args, **kwargs))

    def execute_rank_zero(self, method_name: str, *args, **kwargs):
        return self.execute_rank_zero_async(method_name, *args, **kwargs)

    def execute_rank_zero_sync(self, method_name: str, *args, **kwargs):
        return _resolve(self.execute_rank_zero_async(method_name, *args, **kwargs))

    # -- several roles in one process (``base/fused.py``)
    def spawn_fused(self, prefix_set) -> dict:
        from ..base.fused import spawn_fused

        return spawn_fused(self, prefix_set, func_generator)

    def fuse(self, prefix_set):
        from ..base.fused import fuse

        return fuse(self, prefix_set, func_generator)

    @staticmethod
    def _slice_args(i: int, n: int, args, kwargs):
        """Per-worker arguments: lists of length n are split, everything else is broadcast."""
        sa = tuple(a[i] if isinstance(a, list) and len(a) == n else a for a in args)
        sk = {k: (v[i] if isinstance(v, list) and len(v) == n else v) for k, v in kwargs.items()}
        return sa, sk


class InProcessWorkerGroup(_LocalGroupBase):
    def __init__(self, resource_pool: ResourcePool | int = 1, cls_with_init: ClassWithInitArgs = None, **kwargs):
        pool = resource_pool if isinstance(resource_pool, ResourcePool) else ResourcePool([int(resource_pool)])
        super().__init__(pool, cls_with_init, **kwargs)
        n = pool.world_size
        saved = {k: os.environ.get(k) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
        for r in range(n):
            os.environ.update(RANK=str(r), WORLD_SIZE=str(n), LOCAL_RANK=str(r))
            self._workers.append(cls_with_init())
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
        self._bind()

    def _is_worker_alive(self, worker) -> bool:
        return True

    def execute_all_async(self, method_name: str, *args, **kwargs):
        n = len(self._workers)
        out = []
        for i, w in enumerate(self._workers):
            sa, sk = self._slice_args(i, n, args, kwargs)
            out.append(getattr(w, method_name)(*sa, **sk))
        return out

    def execute_rank_zero_async(self, method_name: str, *args, **kwargs):
        return getattr(self._workers[0], method_name)(*args, **kwargs)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker_main(conn, cls_with_init, env: dict):
    os.environ.update(env)
    from ...utils.process import set_death_signal

    set_death_signal()  # a worker never outlives the controller that spawned it
    try:
        if env.get("VERL_WORKER_DEVICE") == "cuda":
            import torch

            torch.cuda.set_device(int(env["LOCAL_RANK"]))
        worker = cls_with_init()
        conn.send(("ready", None))
    except Exception:
        conn.send(("error", traceback.format_exc()))
        return
    while True:
        try:
            msg = conn.recv()
        except EOFError:
            break
        if msg is None:
            break
        name, args, kwargs = msg
        try:
            res = getattr(worker, name)(*args, **kwargs)
            if isinstance(res, DataProto) and res.batch is not None:
                res = res.to("cpu")
            conn.send(("ok", res))
        except Exception:
            conn.send(("error", traceback.format_exc()))


class _PipeFuture:
    def __init__(self, conn, rank: int, name: str):
        self.conn, self.rank, self.name = conn, rank, name
        self._done, self._value = False, None

    def result(self, timeout: Optional[float] = None):
        if not self._done:
            if timeout is not None and not self.conn.poll(timeout):
                raise TimeoutError(f"worker {self.rank} did not answer '{self.name}' within {timeout}s")
            try:
                status, payload = self.conn.recv()
            except EOFError:
                raise RuntimeError(f"worker {self.rank} died while running '{self.name}'") from None
            if status == "error":
                raise RuntimeError(f"worker {self.rank} failed in '{self.name}':\n{payload}")
            self._done, self._value = True, payload
        return self._value


class MultiprocessWorkerGroup(_LocalGroupBase):
    def __init__(self, resource_pool: ResourcePool | int, cls_with_init: ClassWithInitArgs, device: str = "cpu",
                 env: Optional[dict] = None, start_timeout: float = 600.0, **kwargs):
        pool = resource_pool if isinstance(resource_pool, ResourcePool) else ResourcePool([int(resource_pool)])
        super().__init__(pool, cls_with_init, **kwargs)
        n = pool.world_size
        ctx = mp.get_context("spawn")
        self._master_addr, self._master_port = "127.0.0.1", str(_free_port())
        self._conns, self._procs = [], []
        for r in range(n):
            parent, child = ctx.Pipe()
            e = dict(RANK=str(r), WORLD_SIZE=str(n), LOCAL_RANK=str(r), LOCAL_WORLD_SIZE=str(n),
                     MASTER_ADDR=self._master_addr, MASTER_PORT=self._master_port, VERL_WORKER_DEVICE=device)
            if device != "cuda":
                e["VERL_ENGINE_DEVICE"] = "cpu"
            e.update(env or {})
            p = ctx.Process(target=_worker_main, args=(child, cls_with_init, e), daemon=True)
            p.start()
            child.close()
            self._conns.append(parent)
            self._procs.append(p)
            self._workers.append(p)
        for r, c in enumerate(self._conns):
            if not c.poll(start_timeout):
                self.shutdown()
                raise TimeoutError(f"worker {r} did not start within {start_timeout}s")
            status, payload = c.recv()
            if status != "ready":
                self.shutdown()
                raise RuntimeError(f"worker {r} failed to start:\n{payload}")
        self._bind()

    def _is_worker_alive(self, worker) -> bool:
        return worker.is_alive()

    def execute_all_async(self, method_name: str, *args, **kwargs):
        n = len(self._conns)
        futs = []
        for i, c in enumerate(self._conns):
            sa, sk = self._slice_args(i, n, args, kwargs)
            c.send((method_name, sa, sk))
            futs.append(_PipeFuture(c, i, method_name))
        return futs

    def execute_rank_zero_async(self, method_name: str, *args, **kwargs):
        self._conns[0].send((method_name, args, kwargs))
        return _PipeFuture(self._conns[0], 0, method_name)

    def shutdown(self) -> None:
        for c in self._conns:
            try:
                c.send(None)
            except Exception:
                pass
        for p in self._procs:
            p.join(timeout=5)
            if p.is_alive():
                p.kill()

    def __del__(self):
        try:
            self.shutdown()
        except Exception:
            pass


def _resolve(x):  # noqa: F811  (also understands pipe futures)
    if hasattr(x, "result") and callable(x.result):
        return x.result()
    if isinstance(x, list):
        return [_resolve(v) for v in x]
    return x


class SPMDWorkerGroup(_LocalGroupBase):
    """Controller-replicated mode: this process holds exactly one worker; every proxy call runs on it with the
    arguments untouched and returns its result untouched.  The trainer is then responsible for sharding the data
    by rank (it loads only its shard) and for reducing metrics across ranks."""

    is_spmd = True

    def __init__(self, resource_pool=None, cls_with_init: ClassWithInitArgs = None, **kwargs):
        super().__init__(ResourcePool([1]), cls_with_init, **kwargs)
        self._workers.append(cls_with_init())
        for name in dir(cls_with_init.cls):
            from ..base.decorator import MAGIC_ATTR

            try:
                m = getattr(cls_with_init.cls, name)
            except Exception:
                continue
            if callable(m) and hasattr(m, MAGIC_ATTR):
                setattr(self, name, getattr(self._workers[0], name))

    def _is_worker_alive(self, worker) -> bool:
        return True

    @property
    def worker(self):
        return self._workers[0]

    def execute_all_async(self, method_name: str, *args, **kwargs):
        return [getattr(self._workers[0], method_name)(*args, **kwargs)]

    def execute_rank_zero_async(self, method_name: str, *args, **kwargs):
        return getattr(self._workers[0], method_name)(*args, **kwargs)
