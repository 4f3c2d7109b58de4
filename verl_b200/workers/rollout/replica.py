"""Rollout replicas: one replica = one model instance spanning ``tp * dp * pp`` GPUs, addressable by the
server layer; supports hybrid (shares GPUs and weights with the trainer), colocated and standalone modes.

Parity target: ``verl/workers/rollout/replica.py`` (``TokenOutput`` :39, ``RolloutMode`` :54, ``RolloutReplica``
:70-299, registry :302-408).
"""

from __future__ import annotations

import asyncio
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Optional

__all__ = ["TokenOutput", "RolloutMode", "RolloutReplica", "NativeReplica", "RolloutReplicaRegistry", "get_rollout_replica_class"]


@dataclass
class TokenOutput:
    token_ids: list[int]
    log_probs: Optional[list[float]] = None
    routed_experts: Any = None
    stop_reason: Optional[str] = None  # completed | aborted | length | None
    num_preempted: Optional[int] = None
    extra_fields: dict = field(default_factory=dict)


class RolloutMode(Enum):
    HYBRID = "hybrid"          # same process / GPUs as the trainer, weights shared in place
    COLOCATED = "colocated"    # same GPUs, separate engine memory
    STANDALONE = "standalone"  # own GPUs; weights arrive through a checkpoint engine


class RolloutReplica:
    """Lifecycle and control surface of one replica."""

    def __init__(self, replica_rank: int, config, model_config, gpus_per_node: int = 8, is_reward_model: bool = False):
        self.replica_rank = replica_rank
        self.config, self.model_config = config, model_config
        g = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
        self.world_size = int(g("tensor_model_parallel_size", 1)) * int(g("data_parallel_size", 1)) * int(g("pipeline_model_parallel_size", 1))
        self.gpus_per_node = min(gpus_per_node, self.world_size)
        self.nnodes = max(1, self.world_size // self.gpus_per_node)
        self.is_reward_model = is_reward_model
        self.rollout_mode: Optional[RolloutMode] = None
        self.workers: list = []
        self.servers: list = []
        self._server_address: Optional[str] = None
        self._server_handle = None

    async def init_hybrid(self, worker_group, **kwargs):
        self.rollout_mode = RolloutMode.HYBRID
        lo = self.replica_rank * self.world_size
        self.workers = getattr(worker_group, "_workers", [])[lo : lo + self.world_size]
        await self.launch_servers()

    async def init_colocated(self, resource_pool=None, **kwargs):
        self.rollout_mode = RolloutMode.COLOCATED
        await self.launch_servers()

    async def init_standalone(self, **kwargs):
        self.rollout_mode = RolloutMode.STANDALONE
        await self.launch_servers()

    async def launch_servers(self):
        raise NotImplementedError

    @property
    def server_address(self) -> Optional[str]:
        return self._server_address

    @property
    def server_handle(self):
        return self._server_handle

    async def wake_up(self):
        await asyncio.gather(*[s.wake_up() for s in self.servers])

    async def sleep(self):
        await asyncio.gather(*[s.sleep() for s in self.servers])

    async def abort_all_requests(self):
        return await asyncio.gather(*[s.abort_all_requests() for s in self.servers])

    async def resume_generation(self):
        await asyncio.gather(*[s.resume_generation() for s in self.servers])

    async def clear_kv_cache(self):
        await asyncio.gather(*[s.clear_kv_cache() for s in self.servers])

    async def start_profile(self, **kw):
        await asyncio.gather(*[s.start_profile(**kw) for s in self.servers if hasattr(s, "start_profile")])

    async def stop_profile(self):
        await asyncio.gather(*[s.stop_profile() for s in self.servers if hasattr(s, "stop_profile")])


class NativeServer:
    """Async facade over one in-process engine: requests from many coroutines are funnelled into the engine's
    continuous-batching loop, which runs while any request is pending."""

    def __init__(self, engine, max_model_len: int):
        self.engine, self.max_model_len = engine, max_model_len
        self._futures: dict[str, asyncio.Future] = {}
        self._loop_task: Optional[asyncio.Task] = None
        self._paused = False
        self._global_steps = 0

    async def _drive(self):
        while self._futures and not self._paused:
            for out in self.engine.step():
                fut = self._futures.pop(out.request_id, None)
                if fut is not None and not fut.done():
                    fut.set_result(out)
            await asyncio.sleep(0)
        self._loop_task = None

    async def generate(self, prompt_ids: list[int], sampling_params: dict, request_id: str, **kwargs) -> TokenOutput:
        from .native.engine import SamplingParams

        sp = dict(sampling_params or {})
        budget = self.max_model_len - len(prompt_ids) - 1
        mt = sp.pop("max_tokens", sp.pop("max_new_tokens", None))
        mt = budget if mt is None else max(1, min(int(mt), budget))
        params = SamplingParams(temperature=float(sp.get("temperature", 1.0)), top_p=float(sp.get("top_p", 1.0)),
                                top_k=int(sp.get("top_k", -1)), max_tokens=mt, ignore_eos=bool(sp.get("ignore_eos", False)),
                                logprobs=bool(sp.get("logprobs", True)), seed=sp.get("seed"))
        fut = asyncio.get_running_loop().create_future()
        self._futures[request_id] = fut
        self.engine.add_request(prompt_ids, params, request_id=request_id)
        if self._loop_task is None and not self._paused:
            self._loop_task = asyncio.ensure_future(self._drive())
        out = await fut
        return TokenOutput(token_ids=out.token_ids, log_probs=out.log_probs, stop_reason=out.stop_reason,
                           num_preempted=out.num_preempted, extra_fields={"global_steps": self._global_steps})

    async def wake_up(self):
        self.engine.resume_kv_cache()

    async def sleep(self):
        if not self.engine.running:
            self.engine.release_kv_cache()

    async def clear_kv_cache(self):
        self.engine.clear_kv_cache()

    async def abort_all_requests(self):
        """Retire everything in flight with stop_reason 'aborted' (partial outputs are returned to the callers)."""
        self._paused = True
        outs = self.engine.abort()
        for out in self.engine.finished + outs:
            fut = self._futures.pop(out.request_id, None)
            if fut is not None and not fut.done():
                fut.set_result(out)
        self.engine.finished = []
        return len(outs)

    async def resume_generation(self):
        self._paused = False
        if self._futures and self._loop_task is None:
            self._loop_task = asyncio.ensure_future(self._drive())

    async def set_global_steps(self, steps: int):
        self._global_steps = int(steps)


class NativeReplica(RolloutReplica):
    """Replica backed by the in-process native engine of the local worker."""

    def __init__(self, replica_rank, config, model_config, gpus_per_node: int = 8, is_reward_model: bool = False, engine=None):
        super().__init__(replica_rank, config, model_config, gpus_per_node, is_reward_model)
        self._engine = engine

    async def launch_servers(self):
        eng = self._engine
        if eng is None and self.workers:
            eng = getattr(self.workers[0], "rollout", None)
        assert eng is not None, "NativeReplica needs an engine (pass engine= or init_hybrid with in-process workers)"
        srv = NativeServer(eng, eng.max_model_len)
        self.servers = [srv]
        self._server_handle = srv
        self._server_address = f"inproc://replica-{self.replica_rank}"


class RolloutReplicaRegistry:
    _registry: dict[str, Callable[[], type]] = {}

    @classmethod
    def register(cls, name: str, loader: Callable[[], type]) -> None:
        cls._registry[name] = loader

    @classmethod
    def get(cls, name: str) -> type:
        if name not in cls._registry:
            raise ValueError(f"Unknown rollout mode: {name}. Supported backends: {sorted(cls._registry)}")
        return cls._registry[name]()


RolloutReplicaRegistry.register("native", lambda: NativeReplica)


def _http_replica(kind: str):
    def load():
        from . import http_replica

        return http_replica.HTTPReplica if kind == "sglang" else http_replica.OpenAIReplica

    return load


# inference servers that run outside this process and are reached over HTTP (SGLang's native API; OpenAI-compatible
# completion servers such as ``vllm serve`` and ``trtllm-serve``)
for _name, _kind in (("sglang", "sglang"), ("http", "sglang"), ("trtllm", "openai"), ("openai", "openai")):
    RolloutReplicaRegistry.register(_name, _http_replica(_kind))


def get_rollout_replica_class(rollout: str) -> type[RolloutReplica]:
    return RolloutReplicaRegistry.get(rollout)
