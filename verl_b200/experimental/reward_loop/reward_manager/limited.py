"""Rate-limited scoring for reward functions that call a metered external API: a concurrency cap, a requests-per-minute
bucket and a tokens-per-minute bucket, all shared by every instance in the process, plus a per-call timeout.

Parity target: ``.../reward_manager/limited.py`` (``AsyncTokenBucket`` :32-170, ``RateLimitedRewardManager`` :174-540).
"""

from __future__ import annotations

import asyncio
import time
from typing import Optional

from .naive import NaiveRewardManager
from .registry import register

__all__ = ["AsyncTokenBucket", "RateLimitedRewardManager"]


class AsyncTokenBucket:
    """Starts full, refills at ``rate_limit`` tokens/s up to ``max_tokens``; ``acquire(n)`` sleeps until n are there.
    A request larger than the bucket waits for the whole bucket, takes it, and keeps waiting for the rest."""

    def __init__(self, rate_limit: float, max_tokens: Optional[float] = None, clock=time.monotonic, sleep=asyncio.sleep):
        self.rate_limit = float(rate_limit)
        self.max_tokens = float(max_tokens or rate_limit)
        self.tokens = self.max_tokens
        self._clock, self._sleep = clock, sleep
        self._last = clock()
        self._lock = asyncio.Lock()

    def _refill(self) -> None:
        now = self._clock()
        self.tokens = min(self.max_tokens, self.tokens + (now - self._last) * self.rate_limit)
        self._last = now

    async def acquire(self, num_tokens: float = 1.0) -> None:
        need = float(num_tokens)
        while need > 0:
            async with self._lock:
                self._refill()
                take = min(need, self.max_tokens)
                if self.tokens >= take:
                    self.tokens -= take
                    need -= take
                    continue
                wait = (take - self.tokens) / self.rate_limit
            await self._sleep(wait)


@register("rate_limited")
class RateLimitedRewardManager(NaiveRewardManager):
    _semaphore: Optional[asyncio.Semaphore] = None
    _rpm: Optional[AsyncTokenBucket] = None
    _tpm: Optional[AsyncTokenBucket] = None
    _configured = None

    @classmethod
    def configure(cls, max_concurrent: int = 1, max_rpm: Optional[float] = None, max_tpm: Optional[float] = None) -> None:
        key = (max_concurrent, max_rpm, max_tpm)
        if cls._configured == key:
            return
        cls._configured = key
        cls._semaphore = asyncio.Semaphore(int(max_concurrent))
        cls._rpm = AsyncTokenBucket(max_rpm / 60.0, max_rpm / 60.0 if max_rpm >= 60 else 1.0) if max_rpm else None
        cls._tpm = AsyncTokenBucket(max_tpm / 60.0, max_tpm / 60.0) if max_tpm else None

    def __init__(self, config, tokenizer, compute_score=None, **kw):
        super().__init__(config, tokenizer, compute_score, **kw)
        r = config.get("reward") or config.get("reward_model") or {}
        g = r.get if hasattr(r, "get") else (lambda k, d=None: d)
        self.timeout = g("timeout", 300.0)
        self.estimated_tokens = g("estimated_tokens_per_request", 2000)
        self.configure(int(g("max_concurrent", 1) or 1), g("max_rpm"), g("max_tpm"))

    async def run_single(self, data):
        cls = type(self)
        if cls._rpm is not None:
            await cls._rpm.acquire(1.0)
        if cls._tpm is not None:
            await cls._tpm.acquire(float(self.estimated_tokens))
        async with cls._semaphore:
            try:
                return await asyncio.wait_for(super().run_single(data), timeout=self.timeout)
            except asyncio.TimeoutError:
                return {"reward_score": 0.0, "reward_extra_info": {"timeout": True, "acc": 0.0}}
            except Exception as e:
                return {"reward_score": 0.0, "reward_extra_info": {"error": repr(e), "acc": 0.0}}
