"""In-process key/value sample store with tags ("TransferQueue" role of the v1 trainer).

Values are per-key field dictionaries (tensors, lists, scalars); tags are small metadata dictionaries that can be
listed and filtered without touching the values. Keys live in partitions (``train`` / ``val``). All methods are
thread-safe so a producer thread (rollout) and a consumer (trainer) may share one store. A cross-process variant
backed by a ``torch.distributed`` store is in ``verl_b200.experimental.fully_async_policy.message_queue``.

Parity target: the external TransferQueue package as used by ``verl/trainer/ppo/v1/replay_buffer.py`` and
``verl/protocol.py:1231-1331`` (``KVBatchMeta``).
"""

from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable, Optional

__all__ = ["KVBatchMeta", "TransferQueue", "get_default_queue", "tqbridge"]


@dataclass
class KVBatchMeta:
    """Handle on a set of keys (and optionally a subset of fields) of one partition; cheap to pass around."""

    keys: list[str]
    partition_id: str = "train"
    fields: Optional[list[str]] = None
    tags: list[dict] = field(default_factory=list)

    def __len__(self) -> int:
        return len(self.keys)

    def chunk(self, n: int) -> list["KVBatchMeta"]:
        size = (len(self.keys) + n - 1) // n
        return [KVBatchMeta(self.keys[i * size:(i + 1) * size], self.partition_id, self.fields, self.tags[i * size:(i + 1) * size])
                for i in range(n)]

    @staticmethod
    def concat(metas: Iterable["KVBatchMeta"]) -> "KVBatchMeta":
        metas = list(metas)
        out = KVBatchMeta([], metas[0].partition_id if metas else "train", metas[0].fields if metas else None, [])
        for m in metas:
            out.keys += m.keys
            out.tags += m.tags
        return out


class TransferQueue:
    def __init__(self):
        self._lock = threading.RLock()
        self._values: dict[str, dict[str, dict[str, Any]]] = {}
        self._tags: dict[str, dict[str, dict]] = {}
        self._cond = threading.Condition(self._lock)

    def put(self, key: str, fields: Optional[dict] = None, tags: Optional[dict] = None, partition_id: str = "train") -> None:
        with self._cond:
            self._values.setdefault(partition_id, {}).setdefault(key, {}).update(fields or {})
            self._tags.setdefault(partition_id, {}).setdefault(key, {}).update(tags or {})
            self._cond.notify_all()

    def set_tags(self, key: str, tags: dict, partition_id: str = "train") -> None:
        self.put(key, None, tags, partition_id)

    def get_tags(self, key: str, partition_id: str = "train") -> dict:
        with self._lock:
            return dict(self._tags.get(partition_id, {}).get(key, {}))

    def list_keys(self, partition_id: str = "train", where: Optional[Callable[[str, dict], bool]] = None) -> list[str]:
        with self._lock:
            tags = self._tags.get(partition_id, {})
            return [k for k, t in tags.items() if where is None or where(k, t)]

    def get(self, keys: Iterable[str], fields: Optional[list[str]] = None, partition_id: str = "train") -> list[dict]:
        with self._lock:
            part = self._values.get(partition_id, {})
            out = []
            for k in keys:
                v = part[k]
                out.append(dict(v) if fields is None else {f: v[f] for f in fields if f in v})
            return out

    def get_meta(self, keys: Iterable[str], fields=None, partition_id: str = "train") -> KVBatchMeta:
        keys = list(keys)
        with self._lock:
            tags = [dict(self._tags.get(partition_id, {}).get(k, {})) for k in keys]
        return KVBatchMeta(keys, partition_id, fields, tags)

    def get_data(self, meta: KVBatchMeta) -> list[dict]:
        return self.get(meta.keys, meta.fields, meta.partition_id)

    def delete(self, keys: Iterable[str], partition_id: str = "train") -> None:
        with self._lock:
            for k in keys:
                self._values.get(partition_id, {}).pop(k, None)
                self._tags.get(partition_id, {}).pop(k, None)

    def clear(self, partition_id: Optional[str] = None) -> None:
        with self._lock:
            for store in (self._values, self._tags):
                if partition_id is None:
                    store.clear()
                else:
                    store.pop(partition_id, None)

    def size(self, partition_id: str = "train") -> int:
        with self._lock:
            return len(self._tags.get(partition_id, {}))

    def wait(self, predicate: Callable[[], bool], timeout: Optional[float] = None) -> bool:
        with self._cond:
            return self._cond.wait_for(predicate, timeout)

    # ---- persistence (the asynchronous trainers checkpoint what is finished but not yet trained on, and the prompts in flight)
    def save_checkpoint(self, path: str, metadata: Optional[dict] = None) -> None:
        """Every partition's fields and tags into ``path/state.pt`` (written to a temporary name first, so a crash in the
        middle of a save leaves the previous file). Parity target: ``transfer_queue.save_checkpoint`` as used by
        ``verl/trainer/ppo/v1/trainer_base.py:887-960``."""
        import os

        import torch

        os.makedirs(path, exist_ok=True)
        with self._lock:
            state = {"values": {p: {k: dict(v) for k, v in part.items()} for p, part in self._values.items()},
                     "tags": {p: {k: dict(t) for k, t in part.items()} for p, part in self._tags.items()},
                     "metadata": dict(metadata or {})}
        tmp = os.path.join(path, "state.pt.tmp")
        torch.save(state, tmp)
        os.replace(tmp, os.path.join(path, "state.pt"))

    def load_checkpoint(self, path: str) -> dict:
        """Replace the queue's content by a saved state; returns the metadata stored with it."""
        import os

        import torch

        state = torch.load(os.path.join(path, "state.pt"), weights_only=False)
        with self._cond:
            self._values = {p: dict(part) for p, part in state["values"].items()}
            self._tags = {p: dict(part) for p, part in state["tags"].items()}
            self._cond.notify_all()
        return dict(state.get("metadata", {}))


_default: Optional[TransferQueue] = None


def get_default_queue() -> TransferQueue:
    global _default
    if _default is None:
        _default = TransferQueue()
    return _default


# ----------------------------------------------------------------------------------------------- tqbridge
def _is_collecting_worker(dispatch_mode, args) -> bool:
    """Whether the worker that runs the decorated method is the one whose output is kept: with an nd-mesh dispatch only the
    collecting rank of each data-parallel group writes back, so the rows of a replica are not stored several times."""
    if dispatch_mode is None or not args:
        return True
    worker = args[0]
    mesh = dispatch_mode.get("mesh_name") if isinstance(dispatch_mode, dict) else None
    query = getattr(worker, "query_collect_info", None)
    if mesh is None or query is None:
        return True
    try:
        return bool(query(mesh))
    except Exception:
        return True


def _rows_to_batch(rows: list[dict], meta: "KVBatchMeta"):
    """Per-key field dictionaries -> one batch-first tensor dictionary (tensors stacked, the rest as object arrays)."""
    import numpy as np
    import torch

    from .tensordict_lite import TensorDict

    if not rows:
        return TensorDict({}, batch_size=(0,))
    out = {}
    for f in rows[0]:
        vals = [r[f] for r in rows]
        if all(isinstance(v, torch.Tensor) for v in vals) and len({tuple(v.shape) for v in vals}) == 1:
            out[f] = torch.stack(vals)
        else:
            out[f] = np.array(vals, dtype=object)
    return TensorDict(out, batch_size=(len(rows),))


def tqbridge(dispatch_mode=None, queue: Optional["TransferQueue"] = None, put_data: bool = True):
    """Decorator that lets a method written for real batches be called with a :class:`KVBatchMeta` handle instead.

    Every ``KVBatchMeta`` among the arguments is replaced by the batch it names (a batch-first tensor dictionary fetched
    from the queue); the method runs; if it returns a tensor dictionary with one row per key, its fields are written back
    under the same keys and the *handle* is returned (with the new field names added), so the data never travels through
    the controller. Calls without a handle go straight through. Coroutine functions are supported. With ``dispatch_mode``
    only the collecting worker of a data-parallel group writes back (the others return an empty handle).

    Parity target: ``verl/utils/transferqueue_utils.py:347-470``."""
    import asyncio
    import functools

    def find(args, kwargs):
        for v in list(args) + list(kwargs.values()):
            if isinstance(v, KVBatchMeta):
                return v
        return None

    def decorator(func):
        def before(args, kwargs):
            q = queue or get_default_queue()
            meta = find(args, kwargs)
            conv = lambda v: _rows_to_batch(q.get_data(v), v) if isinstance(v, KVBatchMeta) else v
            return q, meta, [conv(a) for a in args], {k: conv(v) for k, v in kwargs.items()}

        def after(q, meta, args, output):
            from .tensordict_lite import TensorDict

            rows = isinstance(output, TensorDict) and len(output.batch_size) > 0 and output.batch_size[0] == len(meta)
            if not (put_data and rows):
                return output
            if not _is_collecting_worker(dispatch_mode, args):
                return KVBatchMeta([], meta.partition_id, meta.fields, [])
            names = list(output.keys())
            for i, key in enumerate(meta.keys):
                q.put(key, {f: output[f][i] for f in names}, partition_id=meta.partition_id)
            fields = None if meta.fields is None else sorted(set(meta.fields) | set(names))
            return KVBatchMeta(list(meta.keys), meta.partition_id, fields, list(meta.tags))

        if asyncio.iscoroutinefunction(func):
            @functools.wraps(func)
            async def inner(*args, **kwargs):
                if find(args, kwargs) is None:
                    return await func(*args, **kwargs)
                q, meta, a2, k2 = before(args, kwargs)
                return after(q, meta, a2, await func(*a2, **k2))
        else:
            @functools.wraps(func)
            def inner(*args, **kwargs):
                if find(args, kwargs) is None:
                    return func(*args, **kwargs)
                q, meta, a2, k2 = before(args, kwargs)
                return after(q, meta, a2, func(*a2, **k2))

        return inner

    return decorator
