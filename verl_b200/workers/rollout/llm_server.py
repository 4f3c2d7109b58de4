"""Server layer: load balancing over replicas and the token-in / token-out client used by agent loops.

Parity target: ``verl/workers/rollout/llm_server.py`` (``GlobalRequestLoadBalancer`` :46-194, ``LLMServerClient``
:197-289, ``FullyAsyncLLMServerClient`` :292-461, ``LLMServerManager`` :464-647).
"""

from __future__ import annotations

import asyncio
import hashlib
from collections import OrderedDict
from typing import Any, Optional

from .replica import RolloutReplica, TokenOutput, get_rollout_replica_class

__all__ = ["GlobalRequestLoadBalancer", "LLMServerClient", "FullyAsyncLLMServerClient", "LLMServerManager"]


class GlobalRequestLoadBalancer:
    """Sticky sessions (LRU map request_id -> server) on top of least-in-flight routing; servers can be added and
    removed at run time (elastic rollout)."""

    def __init__(self, server_ids: list[str], max_cache_size: int = 10000, deterministic: bool = False):
        self._inflight: dict[str, int] = {s: 0 for s in server_ids}
        self._sticky: OrderedDict[str, str] = OrderedDict()
        self._max_cache = max_cache_size
        self._deterministic = deterministic

    def acquire_server(self, request_id: str) -> Optional[str]:
        if not self._inflight:
            return None
        sid = self._sticky.get(request_id)
        if sid is None or sid not in self._inflight:
            if self._deterministic:
                ids = sorted(self._inflight)
                sid = ids[int(hashlib.md5(request_id.encode()).hexdigest(), 16) % len(ids)]
            else:
                sid = min(self._inflight, key=lambda s: (self._inflight[s], s))
            self._sticky[request_id] = sid
            if len(self._sticky) > self._max_cache:
                self._sticky.popitem(last=False)
        else:
            self._sticky.move_to_end(request_id)
        self._inflight[sid] += 1
        return sid

    def release_server(self, server_id: str) -> None:
        if server_id in self._inflight and self._inflight[server_id] > 0:
            self._inflight[server_id] -= 1

    def add_servers(self, server_ids: list[str]) -> None:
        for s in server_ids:
            self._inflight.setdefault(s, 0)

    def remove_servers(self, server_ids: list[str]) -> None:
        for s in server_ids:
            self._inflight.pop(s, None)
        for rid in [r for r, s in self._sticky.items() if s in server_ids]:
            del self._sticky[rid]

    def snapshot(self) -> dict[str, int]:
        return dict(self._inflight)

    def get_total_inflight(self) -> int:
        return sum(self._inflight.values())

    def clear_sticky_cache(self) -> dict:
        """Forget which server each request was pinned to: the next ``acquire_server`` of every request (a retry after an
        abort included) goes to the least-loaded server. Returns what was cleared and the loads at that moment."""
        n = len(self._sticky)
        self._sticky.clear()
        return {"cleared_entries": n, "server_loads": dict(self._inflight)}


class LLMServerClient:
    """``generate(request_id, prompt_ids, sampling_params) -> TokenOutput`` against the balanced replicas."""

    def __init__(self, config, servers: dict[str, Any], load_balancer: GlobalRequestLoadBalancer):
        self.config, self.servers, self.lb = config, servers, load_balancer

    def _cap(self, prompt_len: int, sampling_params: dict) -> dict:
        g = self.config.get if hasattr(self.config, "get") else (lambda k, d=None: getattr(self.config, k, d))
        resp, prm = int(g("response_length", 512)), int(g("prompt_length", 512))
        sp = dict(sampling_params)
        default = min(resp, prm + resp - prompt_len)
        mt = sp.pop("max_new_tokens", sp.get("max_tokens", default))
        sp["max_tokens"] = max(1, min(int(mt), prm + resp - prompt_len if prm + resp > prompt_len else 1))
        return sp

    async def generate(self, request_id: str, *, prompt_ids: list[int], sampling_params: dict, **kwargs) -> TokenOutput:
        sid = self.lb.acquire_server(request_id)
        if sid is None:
            raise RuntimeError("no rollout server available")
        try:
            return await self.servers[sid].generate(prompt_ids=prompt_ids, sampling_params=self._cap(len(prompt_ids), sampling_params),
                                                    request_id=request_id, **kwargs)
        finally:
            self.lb.release_server(sid)


class FullyAsyncLLMServerClient(LLMServerClient):
    """Survives aborts: an aborted partial output is kept and generation continues (possibly on another replica,
    with new weights) with the remaining token budget until the request completes."""

    def __init__(self, *a, retry_interval: float = 0.05, max_retries: int = 10000, **k):
        super().__init__(*a, **k)
        self.retry_interval, self.max_retries = retry_interval, max_retries

    async def generate(self, request_id: str, *, prompt_ids: list[int], sampling_params: dict, **kwargs) -> TokenOutput:
        sp = self._cap(len(prompt_ids), sampling_params)
        budget = sp["max_tokens"]
        acc_ids: list[int] = []
        acc_lp: list[float] = []
        extra: dict = {}
        tries = 0
        while True:
            sid = self.lb.acquire_server(request_id)
            if sid is None:
                tries += 1
                if tries > self.max_retries:
                    raise RuntimeError("no rollout server became available")
                await asyncio.sleep(self.retry_interval)
                continue
            try:
                step_sp = dict(sp, max_tokens=budget - len(acc_ids))
                out = await self.servers[sid].generate(prompt_ids=prompt_ids + acc_ids, sampling_params=step_sp,
                                                       request_id=f"{request_id}#{tries}", **kwargs)
            finally:
                self.lb.release_server(sid)
            acc_ids += out.token_ids
            acc_lp += out.log_probs or []
            extra.update(out.extra_fields or {})
            if out.stop_reason != "aborted" or len(acc_ids) >= budget:
                return TokenOutput(acc_ids, acc_lp or None, out.routed_experts, out.stop_reason if out.stop_reason != "aborted" else "length",
                                   tries, extra)
            tries += 1
            await asyncio.sleep(self.retry_interval)


class LLMServerManager:
    """Creates the replicas, the balancer and hands out clients."""

    def __init__(self, config, replicas: list[RolloutReplica], fully_async: bool = False):
        self.config, self.replicas, self.fully_async = config, replicas, fully_async
        self.servers = {r.server_address: r.server_handle for r in replicas}
        self.lb = GlobalRequestLoadBalancer(list(self.servers))

    @classmethod
    async def create(cls, config, worker_group=None, model_config=None, engines: Optional[list] = None, fully_async: bool = False):
        g = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
        replica_cls = get_rollout_replica_class(g("name", "native"))
        replicas = []
        urls = list(g("server_urls", None) or [])
        if urls and engines is None and g("name", "native") in ("sglang", "trtllm", "openai", "http"):
            # servers that already run elsewhere: one replica per address, nothing to launch
            for i in range(len(urls)):
                r = replica_cls(i, config, model_config)
                await r.init_standalone()
                replicas.append(r)
        elif engines is not None:
            for i, eng in enumerate(engines):
                r = replica_cls(i, config, model_config, engine=eng)
                await r.init_standalone()
                replicas.append(r)
        else:
            ws = worker_group.world_size
            per = int(g("tensor_model_parallel_size", 1)) * int(g("data_parallel_size", 1)) * int(g("pipeline_model_parallel_size", 1))
            for i in range(max(1, ws // per)):
                r = replica_cls(i, config, model_config)
                await r.init_hybrid(worker_group)
                replicas.append(r)
        return cls(config, replicas, fully_async)

    def client(self) -> LLMServerClient:
        kind = FullyAsyncLLMServerClient if self.fully_async else LLMServerClient
        return kind(self.config, self.servers, self.lb)

    async def add_replicas(self, replicas: list[RolloutReplica]) -> None:
        for r in replicas:
            self.replicas.append(r)
            self.servers[r.server_address] = r.server_handle
        self.lb.add_servers([r.server_address for r in replicas])

    async def remove_replicas(self, replicas: list[RolloutReplica]) -> None:
        ids = [r.server_address for r in replicas]
        self.lb.remove_servers(ids)
        for r in replicas:
            await r.abort_all_requests()
            self.servers.pop(r.server_address, None)
            if r in self.replicas:
                self.replicas.remove(r)

    async def wake_up(self):
        await asyncio.gather(*[r.wake_up() for r in self.replicas])

    async def sleep(self):
        await asyncio.gather(*[r.sleep() for r in self.replicas])

    async def clear_kv_cache(self):
        await asyncio.gather(*[r.clear_kv_cache() for r in self.replicas])
