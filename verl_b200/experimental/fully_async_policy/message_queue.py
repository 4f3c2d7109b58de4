"""Sample queues between rollout producers and the trainer.

``MessageQueue`` is the in-process bounded queue (oldest sample dropped when full, staleness bookkeeping by weight
version). ``StoreMessageQueue`` gives the same put/get contract across processes on top of the key-value store that
``torch.distributed`` already runs for rendez-vous (no extra service): producers append under a ticket taken with an
atomic add, consumers claim tickets the same way, so any number of producers and consumers may share one queue.

Parity target: ``verl/experimental/fully_async_policy/message_queue.py:55-105`` (``put_sample`` / ``get_sample`` /
``update_param_version`` / ``get_statistics``), which the reference hosts in a Ray actor.
"""

from __future__ import annotations

import pickle
import threading
import time
from collections import deque
from datetime import timedelta
from typing import Any, Optional

__all__ = ["MessageQueue", "StoreMessageQueue", "QueueClosed"]


class QueueClosed(Exception):
    pass


class MessageQueue:
    def __init__(self, max_queue_size: int = 1024, staleness_threshold: Optional[int] = None):
        self.max_queue_size = int(max_queue_size)
        self.staleness_threshold = staleness_threshold
        self._q: deque = deque()
        self._cond = threading.Condition()
        self.current_param_version = 0
        self.total_produced = self.total_consumed = self.dropped_samples = 0
        self._closed = False

    def put_sample(self, sample: Any, param_version: int) -> bool:
        with self._cond:
            if self._closed:
                return False
            if self.staleness_threshold is not None and self.current_param_version - param_version > self.staleness_threshold:
                self.dropped_samples += 1
                return False
            if len(self._q) >= self.max_queue_size:
                self._q.popleft()
                self.dropped_samples += 1
            self._q.append((sample, int(param_version)))
            self.total_produced += 1
            self._cond.notify()
            return True

    def get_sample(self, timeout: Optional[float] = None):
        """(sample, remaining queue length) or ``None`` after ``timeout`` / when closed and empty."""
        with self._cond:
            ok = self._cond.wait_for(lambda: self._q or self._closed, timeout)
            if not ok or not self._q:
                return None
            sample, _ = self._q.popleft()
            self.total_consumed += 1
            return sample, len(self._q)

    def update_param_version(self, version: int) -> None:
        with self._cond:
            self.current_param_version = int(version)

    def get_queue_size(self) -> int:
        with self._cond:
            return len(self._q)

    def get_statistics(self) -> dict:
        with self._cond:
            return {"queue_size": len(self._q), "total_produced": self.total_produced, "total_consumed": self.total_consumed,
                    "dropped_samples": self.dropped_samples, "current_param_version": self.current_param_version,
                    "staleness_threshold": self.staleness_threshold, "max_queue_size": self.max_queue_size}

    def snapshot(self) -> list:
        """The queued ``(sample, parameter version)`` pairs, oldest first (for a checkpoint; the queue is left as it is)."""
        with self._cond:
            return list(self._q)

    def restore(self, items: list) -> None:
        """Put checkpointed pairs back in front of whatever is queued, oldest first."""
        with self._cond:
            self._q.extendleft(reversed([(s, int(v)) for s, v in items]))
            self._cond.notify_all()

    def clear_queue(self) -> None:
        with self._cond:
            self._q.clear()

    def shutdown(self) -> None:
        with self._cond:
            self._closed = True
            self._cond.notify_all()


class StoreMessageQueue:
    """Multi-producer / multi-consumer FIFO over a ``torch.distributed`` store.

    Keys: ``{name}/tail`` (tickets handed to producers), ``{name}/head`` (tickets handed to consumers),
    ``{name}/item/{i}`` (payload). A consumer that claimed a ticket whose payload has not arrived keeps the claim and
    returns ``None``; its next call waits for the same ticket, so no item is ever skipped."""

    def __init__(self, store, name: str):
        self.store, self.name = store, name
        self._claim: Optional[int] = None

    def _count(self, key: str, inc: int = 0) -> int:
        return int(self.store.add(f"{self.name}/{key}", inc))

    def put(self, obj: Any) -> int:
        i = self._count("tail", 1) - 1
        self.store.set(f"{self.name}/item/{i}", pickle.dumps(obj))
        return i

    def qsize(self) -> int:
        return max(0, self._count("tail") - self._count("head"))

    def try_get(self, timeout: float = 0.05) -> Optional[Any]:
        if self._claim is None:
            if self._count("tail") <= self._count("head"):
                return None
            self._claim = self._count("head", 1) - 1
        key = f"{self.name}/item/{self._claim}"
        try:
            self.store.wait([key], timedelta(seconds=max(timeout, 1e-3)))
        except Exception:
            return None  # not there yet: keep the claim
        obj = pickle.loads(self.store.get(key))
        try:
            self.store.delete_key(key)
        except Exception:
            pass
        self._claim = None
        return obj

    def get(self, timeout: float = 60.0, poll: float = 0.05) -> Optional[Any]:
        t0 = time.time()
        while time.time() - t0 < timeout:
            obj = self.try_get(poll)
            if obj is not None:
                return obj
            if self._claim is None:
                time.sleep(poll)
        return None
