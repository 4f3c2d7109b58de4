"""Moves fresh weights from the trainer to the rollout replicas and tells everyone the new version.

In the colocated layout the rollout engine reads the trainer's buffer in place, so a sync is: pause generation
(partial outputs kept) -> clear cached KV -> bump the version -> resume. With a separate rollout pool the same steps
wrap a checkpoint-engine transfer. Parity target: ``verl/experimental/fully_async_policy/param_sync.py``.
"""

from __future__ import annotations

import time
from typing import Callable, Optional

__all__ = ["ParameterSynchronizer"]


class ParameterSynchronizer:
    def __init__(self, pause_fn: Callable[[], None], resume_fn: Callable[[], None], transfer_fn: Callable[[int], dict],
                 message_queue=None, set_version_fn: Optional[Callable[[int], None]] = None):
        self.pause_fn, self.resume_fn, self.transfer_fn = pause_fn, resume_fn, transfer_fn
        self.mq, self.set_version_fn = message_queue, set_version_fn
        self.current_version = 0
        self.last_sync_s = 0.0

    def sync_weights(self, version: int, validate: bool = False) -> dict:
        t0 = time.time()
        self.pause_fn()
        res = self.transfer_fn(version)
        if isinstance(res, (list, tuple)):  # worker groups answer with one entry per worker
            res = res[0] if res else {}
        stats = dict(res or {})
        self.current_version = int(version)
        if self.mq is not None:
            self.mq.update_param_version(self.current_version)
        if self.set_version_fn is not None:
            self.set_version_fn(self.current_version)
        self.resume_fn()
        self.last_sync_s = time.time() - t0
        stats["timing_s/param_sync"] = self.last_sync_s
        return stats
