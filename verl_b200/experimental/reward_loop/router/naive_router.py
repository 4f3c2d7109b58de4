"""Least-loaded dispatch of scoring requests over reward-model servers, with retry on another server when one fails.
Parity target: ``verl/experimental/reward_loop/router/naive_router.py`` (an HTTP proxy in the reference; the servers
here are in-process handles)."""
from __future__ import annotations

import itertools

__all__ = ["NaiveRouter"]


class NaiveRouter:
    def __init__(self, servers: list, max_retries: int = 2):
        assert servers, "router needs at least one server"
        self.servers = list(servers)
        self.inflight = [0] * len(servers)
        self.failures = [0] * len(servers)
        self.max_retries = max_retries
        self._rr = itertools.count()

    def _pick(self, exclude: set) -> int:
        cands = [i for i in range(len(self.servers)) if i not in exclude] or list(range(len(self.servers)))
        low = min(self.inflight[i] for i in cands)
        ties = [i for i in cands if self.inflight[i] == low]
        return ties[next(self._rr) % len(ties)]

    async def score(self, token_ids: list[int], **kw) -> float:
        tried: set = set()
        last = None
        for _ in range(self.max_retries + 1):
            i = self._pick(tried)
            self.inflight[i] += 1
            try:
                return await self.servers[i].score(token_ids, **kw)
            except Exception as e:  # try the next server
                last = e
                self.failures[i] += 1
                tried.add(i)
            finally:
                self.inflight[i] -= 1
        raise RuntimeError(f"all reward servers failed: {last!r}")
