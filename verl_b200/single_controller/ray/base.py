"""Ray back-end of the single-controller runtime (optional: needs the ``ray`` package, which this build does not
ship; the in-process, multi-process and SPMD groups in ``single_controller.local`` are the tested back-ends).

One actor per GPU, placed with placement groups (one bundle per GPU, ``STRICT_PACK`` per node); rank, world size,
master address/port and local rank travel as environment variables; a decorated worker method called on the group
dispatches its arguments with the method's ``dispatch_fn``, calls every actor and collects with ``collect_fn``.

Parity target: ``verl/single_controller/ray/base.py`` (``RayResourcePool`` :105-215, ``RayClassWithInitArgs`` :232-300,
``RayWorkerGroup`` :303-850, ``create_colocated_worker_cls`` :893-960).
"""

from __future__ import annotations

import os
import socket
from typing import Any, Optional

from ..base.decorator import MAGIC_ATTR, Execute, get_predefined_dispatch_fn, get_predefined_execute_fn
from ..base.worker_group import ClassWithInitArgs, ResourcePool, WorkerGroup

__all__ = ["RayResourcePool", "RayClassWithInitArgs", "RayWorkerGroup", "create_colocated_worker_cls", "create_colocated_worker_cls_fused"]


def _ray():
    try:
        import ray

        return ray
    except ImportError as e:
        raise ImportError("trainer.worker_group=ray needs the 'ray' package; use spmd (torchrun), multiprocess or inprocess") from e


class RayResourcePool(ResourcePool):
    def __init__(self, process_on_nodes=None, use_gpu: bool = True, name_prefix: str = "", max_colocate_count: int = 10,
                 detached: bool = False, accelerator_type: Optional[str] = None):
        super().__init__(process_on_nodes, max_colocate_count)
        self.use_gpu, self.name_prefix, self.detached, self.accelerator_type = use_gpu, name_prefix, detached, accelerator_type
        self.pgs = None

    def get_placement_groups(self, strategy: str = "STRICT_PACK", name: Optional[str] = None, device_name: str = "cuda"):
        if self.pgs is not None:
            return self.pgs
        ray = _ray()
        from ray.util.placement_group import placement_group

        bundle = {"CPU": self.max_colocate_count}
        if self.use_gpu:
            bundle["GPU"] = 1
        pgs = [placement_group([dict(bundle) for _ in range(n)], strategy=strategy, name=f"{self.name_prefix}pg_{i}",
                               lifetime="detached" if self.detached else None) for i, n in enumerate(self._store)]
        ray.get([pg.ready() for pg in pgs])
        self.pgs = pgs
        return pgs


class RayClassWithInitArgs(ClassWithInitArgs):
    def __init__(self, cls, *args, **kwargs):
        super().__init__(cls, *args, **kwargs)
        self._options: dict = {}
        self._additional_resource: dict = {}

    def set_additional_resource(self, additional_resource: dict) -> None:
        self._additional_resource = additional_resource

    def update_options(self, options: dict) -> None:
        self._options.update(options)

    def __call__(self, placement_group, placement_group_bundle_idx: int, use_gpu: bool = True, num_gpus: float = 1,
                 sharing_with=None, device_name: str = "cuda"):
        ray = _ray()
        from ray.util.scheduling_strategies import PlacementGroupSchedulingStrategy

        opts = {"scheduling_strategy": PlacementGroupSchedulingStrategy(placement_group=placement_group,
                                                                        placement_group_bundle_index=placement_group_bundle_idx)}
        opts.update(self._options)
        if use_gpu:
            opts["num_gpus"] = num_gpus
        if self._additional_resource:
            opts["resources"] = dict(self._additional_resource)
        remote_cls = self.cls if hasattr(self.cls, "remote") else ray.remote(self.cls)
        return remote_cls.options(**opts).remote(*self.args, **self.kwargs)


class RayWorkerGroup(WorkerGroup):
    def __init__(self, resource_pool: Optional[RayResourcePool] = None, ray_cls_with_init: Optional[RayClassWithInitArgs] = None,
                 bin_pack: bool = True, name_prefix: Optional[str] = None, detached: bool = False, worker_names=None,
                 worker_handles=None, device_name: str = "cuda", **kwargs):
        super().__init__(resource_pool=resource_pool, **kwargs)
        self.ray_cls_with_init = ray_cls_with_init
        self.name_prefix = name_prefix or "verl_b200"
        self.device_name = device_name
        self._worker_names: list[str] = []
        if worker_handles is not None:
            self._workers = list(worker_handles)
            self._world_size = len(self._workers)
        elif resource_pool is not None:
            self._init_with_resource_pool(resource_pool, ray_cls_with_init, bin_pack, detached)
        if ray_cls_with_init is not None:
            self._bind_worker_method(ray_cls_with_init.cls)

    def _is_worker_alive(self, worker) -> bool:
        ray = _ray()
        try:
            st = ray.state.actors(worker._actor_id.hex())
            return st.get("State", "ALIVE") == "ALIVE" if st else False
        except Exception:
            return True

    def _init_with_resource_pool(self, pool: RayResourcePool, cls_init: RayClassWithInitArgs, bin_pack: bool, detached: bool) -> None:
        ray = _ray()
        pgs = pool.get_placement_groups(strategy="STRICT_PACK" if bin_pack else "PACK", device_name=self.device_name)
        world = pool.world_size
        self._world_size = world
        rank = -1
        master = {}
        for pg_idx, (pg, n_local) in enumerate(zip(pgs, pool.store)):
            for local_rank in range(n_local):
                rank += 1
                env = {"WORLD_SIZE": str(world), "RANK": str(rank), "LOCAL_RANK": str(local_rank), "LOCAL_WORLD_SIZE": str(n_local),
                       "WG_PREFIX": self.name_prefix, "WG_BACKEND": "ray"}
                if rank != 0:
                    env.update(master)
                name = f"{self.name_prefix}{cls_init.cls.__name__}_{pg_idx}:{local_rank}"
                cls_init.update_options({"runtime_env": {"env_vars": env}, "name": name, **({"lifetime": "detached"} if detached else {})})
                w = cls_init(placement_group=pg, placement_group_bundle_idx=local_rank, use_gpu=pool.use_gpu, device_name=self.device_name)
                self._workers.append(w)
                self._worker_names.append(name)
                if rank == 0:
                    addr, port = ray.get(w._get_node_ip_and_free_port.remote()) if hasattr(w, "_get_node_ip_and_free_port") else (socket.gethostbyname(socket.gethostname()), "29500")
                    master = {"MASTER_ADDR": str(addr), "MASTER_PORT": str(port)}

    def _bind_worker_method(self, user_cls) -> None:
        ray = _ray()
        for name in dir(user_cls):
            try:
                m = getattr(user_cls, name)
            except Exception:
                continue
            if not callable(m) or not hasattr(m, MAGIC_ATTR):
                continue
            attrs = getattr(m, MAGIC_ATTR)
            mode, execute_mode, blocking = attrs["dispatch_mode"], attrs["execute_mode"], attrs["blocking"]
            fns = mode if isinstance(mode, dict) else get_predefined_dispatch_fn(mode)
            dispatch_fn, collect_fn = fns["dispatch_fn"], fns["collect_fn"]
            exec_name = get_predefined_execute_fn(execute_mode)["execute_fn_name"] if not isinstance(execute_mode, str) else execute_mode

            def make(name=name, dispatch_fn=dispatch_fn, collect_fn=collect_fn, exec_name=exec_name, blocking=blocking):
                def call(*args, **kwargs):
                    a, k = dispatch_fn(self, *args, **kwargs)
                    out = getattr(self, exec_name)(name, *a, **k)
                    if blocking:
                        out = ray.get(out)
                    return collect_fn(self, out)

                return call

            setattr(self, name, make())

    # ---- execution primitives
    def execute_rank_zero_async(self, method_name: str, *args, **kwargs):
        return getattr(self._workers[0], method_name).remote(*args, **kwargs)

    def execute_rank_zero_sync(self, method_name: str, *args, **kwargs):
        return _ray().get(self.execute_rank_zero_async(method_name, *args, **kwargs))

    execute_rank_zero = execute_rank_zero_async

    def execute_all_async(self, method_name: str, *args, **kwargs):
        n = len(self._workers)
        sharded = all(isinstance(a, list) and len(a) == n for a in args) and all(isinstance(v, list) and len(v) == n for v in kwargs.values())
        if sharded and (args or kwargs):
            return [getattr(w, method_name).remote(*[a[i] for a in args], **{k: v[i] for k, v in kwargs.items()}) for i, w in enumerate(self._workers)]
        return [getattr(w, method_name).remote(*args, **kwargs) for w in self._workers]

    def execute_all_sync(self, method_name: str, *args, **kwargs):
        return _ray().get(self.execute_all_async(method_name, *args, **kwargs))

    execute_all = execute_all_async

    def spawn(self, prefix_set) -> dict:
        """One view of the same actors per role prefix (methods ``{prefix}_{name}`` appear as ``{name}``)."""
        out = {}
        for prefix in prefix_set:
            g = RayWorkerGroup(worker_handles=self._workers, ray_cls_with_init=self.ray_cls_with_init, name_prefix=self.name_prefix)
            for name in dir(g):
                if name.startswith(prefix + "_"):
                    setattr(g, name[len(prefix) + 1:], getattr(g, name))
            out[prefix] = g
        return out

    @property
    def worker_names(self) -> list[str]:
        return self._worker_names


def create_colocated_worker_cls_fused(class_dict: dict[str, RayClassWithInitArgs]):
    """Fused form of ``create_colocated_worker_cls``: the roles keep their own method names and are addressed through
    per-role views (``RayWorkerGroup.spawn_fused`` / ``fuse``); the generated worker class comes from ``base/fused.py``."""
    from ..base.fused import _build_fused_cls

    import ray

    cia = RayClassWithInitArgs(cls=ray.remote(_build_fused_cls(class_dict)))
    cia.fused_worker_used = True
    cia.raw_cls_dict = {name: c.cls for name, c in class_dict.items()}
    return cia


def create_colocated_worker_cls(class_dict: dict[str, RayClassWithInitArgs]):
    """One actor class hosting several role workers in one process; role methods are exposed as ``{role}_{method}``."""
    first = next(iter(class_dict.values()))

    class WorkerDict(first.cls.__mro__[-2] if len(first.cls.__mro__) > 1 else object):  # common Worker base
        def __init__(self):
            try:
                super().__init__()
            except TypeError:
                pass
            self.worker_dict = {k: v.cls(*v.args, **v.kwargs) for k, v in class_dict.items()}

    for role, ci in class_dict.items():
        for name in dir(ci.cls):
            try:
                m = getattr(ci.cls, name)
            except Exception:
                continue
            if callable(m) and hasattr(m, MAGIC_ATTR):
                def make(role=role, name=name, m=m):
                    def fn(self, *a, **k):
                        return getattr(self.worker_dict[role], name)(*a, **k)

                    setattr(fn, MAGIC_ATTR, getattr(m, MAGIC_ATTR))
                    return fn

                setattr(WorkerDict, f"{role}_{name}", make())
    return RayClassWithInitArgs(cls=WorkerDict)
