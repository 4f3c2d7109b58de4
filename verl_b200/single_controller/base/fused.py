"""Several worker roles in one process, each addressed through its own worker-group view.

``create_colocated_worker_cls_fused({"actor": cia, "critic": cia})`` returns the class (with its constructor arguments) of
a *fused worker*: one process per rank that builds every role's worker, lets them see each other
(``worker.fused_worker_dict``) and runs ``role.method`` when asked for ``"{role}_fwmn_{method}"`` through
``_fuw_execute``. A worker group built from it gives one view per role (``spawn_fused`` / ``fuse``): the view carries the
proxies of that role's ``@register``-ed methods and forwards them to the shared processes, so the controller code written
for separate worker groups runs unchanged on colocated ones. Independent of the process backend (in-process, pipes, Ray).

Parity target: ``verl/single_controller/ray/base.py:749-771`` (``spawn_fused`` / ``fuse``), ``:1030-1130``
(``create_colocated_worker_raw_cls`` / ``FusedWorker``).
"""

from __future__ import annotations

import copy
import os
from contextlib import contextmanager

from .worker import Worker
from .worker_group import ClassWithInitArgs, WorkerGroup

__all__ = ["FusedWorkerCLSName", "create_colocated_worker_cls_fused", "FusedGroupView", "spawn_fused", "fuse"]

FusedWorkerCLSName = "FusedWorker"
_SEP = "_fwmn_"  # "fused worker method name"


@contextmanager
def _temp_env(key: str, value: str):
    old = os.environ.get(key)
    os.environ[key] = value
    try:
        yield
    finally:
        if old is None:
            os.environ.pop(key, None)
        else:
            os.environ[key] = old


class FusedClassWithInitArgs(ClassWithInitArgs):
    """The fused worker class is generated per process (a generated class cannot be pickled to a worker process): what
    travels is the role -> (class, arguments) table, the class is rebuilt on first use on either side."""

    def __init__(self, class_dict: dict[str, ClassWithInitArgs]):
        self.class_dict = class_dict
        self._built = None
        super().__init__(None)
        self.fused_worker_used = True

    @property
    def cls(self):
        if self._built is None:
            self._built = _build_fused_cls(self.class_dict)
        return self._built

    @cls.setter
    def cls(self, value):  # the base constructor assigns it; the generated class replaces whatever is put here
        pass

    def __getstate__(self):
        d = dict(self.__dict__)
        d["_built"] = None
        return d

    def __call__(self, *args, **kwargs):
        return self.cls()


def create_colocated_worker_cls_fused(class_dict: dict[str, ClassWithInitArgs]) -> ClassWithInitArgs:
    return FusedClassWithInitArgs(class_dict)


def _build_fused_cls(class_dict: dict[str, ClassWithInitArgs]):
    raw = {name: cia.cls for name, cia in class_dict.items()}
    init_args = {name: (cia.args, cia.kwargs) for name, cia in class_dict.items()}
    renamed = "_".join([FusedWorkerCLSName] + list(class_dict))

    class FusedWorker(Worker):
        is_fused_worker = True
        raw_cls_dict = raw

        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            self.cls_names = list(raw)
            self.fused_worker_dict = {}
            for name, cls in raw.items():
                a, k = init_args[name]
                with _temp_env("DISABLE_WORKER_INIT", "1"):  # the process is set up once, by the fused worker itself
                    self.fused_worker_dict[name] = cls(*a, **k)
                setattr(self, name, self.fused_worker_dict[name])
            for w in self.fused_worker_dict.values():  # the roles can reach each other (weight sharing, hand-overs)
                setattr(w, Worker.fused_worker_attr_name, self.fused_worker_dict)

        def _fuw_execute(self, method_name: str, *args, **kwargs):
            role, _, method = method_name.partition(_SEP)
            assert role in self.fused_worker_dict and method, f"'{method_name}': no role '{role}' in this fused worker"
            return getattr(self.fused_worker_dict[role], method)(*args, **kwargs)

        # dispatch-mesh queries of a view land on the role that registered the mesh
        def _role_of_mesh(self, mesh_name: str):
            for w in self.fused_worker_dict.values():
                if mesh_name in w._dispatch_mesh:
                    return w
            raise AssertionError(f"{mesh_name} is not registered by any role of {type(self).__name__}")

        def _query_dispatch_info(self, mesh_name: str):
            return self._role_of_mesh(mesh_name)._dispatch_mesh[mesh_name][0]

        def _query_collect_info(self, mesh_name: str):
            return self._role_of_mesh(mesh_name)._dispatch_mesh[mesh_name][1]

    return type(renamed, (FusedWorker,), {})


class FusedGroupView(WorkerGroup):
    """The methods of one role of a fused worker group. Shares the processes of ``parent``; every call goes through the
    parent's execution primitives as ``_fuw_execute("{role}_fwmn_{method}", ...)``."""

    def __init__(self, parent: WorkerGroup, role: str, role_cls, func_generator):
        self.__dict__.update({k: v for k, v in parent.__dict__.items() if not callable(v) or k.startswith("_")})
        self._parent, self.sub_cls_name, self.fused_worker_used = parent, role, True
        self._dispatch_info, self._collect_info = {}, {}
        self.method_names = self._bind_worker_method(role_cls, func_generator)

    def _name(self, method_name: str) -> tuple[str, tuple]:
        if method_name in ("_query_dispatch_info", "_query_collect_info"):
            return method_name, ()
        return WorkerGroup.fused_worker_execute_fn_name, (f"{self.sub_cls_name}{_SEP}{method_name}",)

    def _forward(self, prim: str, method_name: str, *args, **kwargs):
        name, lead = self._name(method_name)
        return getattr(self._parent, prim)(name, *lead, *args, **kwargs)

    def execute_all(self, m, *a, **k):
        return self._forward("execute_all", m, *a, **k)

    def execute_all_sync(self, m, *a, **k):
        return self._forward("execute_all_sync", m, *a, **k)

    def execute_all_async(self, m, *a, **k):
        return self._forward("execute_all_async", m, *a, **k)

    def execute_rank_zero(self, m, *a, **k):
        return self._forward("execute_rank_zero", m, *a, **k)

    def execute_rank_zero_sync(self, m, *a, **k):
        return self._forward("execute_rank_zero_sync", m, *a, **k)

    def execute_rank_zero_async(self, m, *a, **k):
        return self._forward("execute_rank_zero_async", m, *a, **k)

    @property
    def world_size(self) -> int:
        return self._parent.world_size


def spawn_fused(group: WorkerGroup, prefix_set, func_generator) -> dict[str, FusedGroupView]:
    """One view per role of the fused worker class that ``group`` was built from."""
    raw = getattr(group.cls_with_init.cls, "raw_cls_dict", None)
    assert raw is not None, "spawn_fused needs a worker group built from create_colocated_worker_cls_fused"
    return {role: FusedGroupView(group, role, raw[role], func_generator) for role in prefix_set}


def fuse(group: WorkerGroup, prefix_set, func_generator) -> WorkerGroup:
    """Attach the views as attributes: ``group.actor.update_actor(...)``, ``group.critic.compute_values(...)``."""
    group.wg_dict = spawn_fused(group, prefix_set, func_generator)
    for role, view in group.wg_dict.items():
        setattr(group, role, view)
    return group
