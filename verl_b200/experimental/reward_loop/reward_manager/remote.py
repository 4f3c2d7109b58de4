"""Scores in a pool of worker processes, so heavy CPU rules (symbolic math, code execution) leave the event loop and
the GIL of the rollout driver alone. Parity target: ``.../reward_manager/remote.py`` (the reference uses Ray actors)."""
from __future__ import annotations

import asyncio
import concurrent.futures as cf

from .naive import NaiveRewardManager
from .registry import register

__all__ = ["RemoteRewardManager"]

_POOL = None


def _pool(workers: int):
    global _POOL
    if _POOL is None:
        _POOL = cf.ProcessPoolExecutor(max_workers=workers)
    return _POOL


def _call(fn, kw):
    return fn(**kw)


@register("remote")
class RemoteRewardManager(NaiveRewardManager):
    def __init__(self, config, tokenizer, compute_score=None, num_workers: int = 8, **kw):
        super().__init__(config, tokenizer, compute_score, **kw)
        self.num_workers = num_workers

    async def _score(self, **kw):
        if self.is_async_reward_score:
            return await self.compute_score(**kw)
        kw = {k: v for k, v in kw.items() if k != "extra_info"} | {"extra_info": {k: v for k, v in (kw.get("extra_info") or {}).items()
                                                                                 if isinstance(v, (int, float, str, bool, type(None)))}}
        return await asyncio.get_running_loop().run_in_executor(_pool(self.num_workers), _call, self.compute_score, kw)
