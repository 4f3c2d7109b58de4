"""``@register`` and the dispatch / collect modes of the single-controller programming model.

A worker method decorated with ``@register(dispatch_mode=...)`` gets a driver-side proxy on the worker group:
the proxy splits the arguments for the workers (dispatch), runs the method on them (execute) and merges the
results (collect).

Parity target: ``verl/single_controller/base/decorator.py`` (``Dispatch`` :38-47, ``Execute`` :61-63,
dispatch/collect functions :120-304, registry :308-338, ``register`` :398-444).
"""

from __future__ import annotations

import inspect
from functools import partial, wraps
from typing import Any, Callable

from ...protocol import DataProto, DataProtoFuture, BatchData
from ...utils.tensordict_lite import TensorDict, cat_tensordicts, chunk_tensordict

__all__ = ["Dispatch", "Execute", "register", "MAGIC_ATTR", "get_predefined_dispatch_fn", "get_predefined_execute_fn",
           "register_dispatch_mode", "update_dispatch_mode", "init_predefined_dispatch_mode", "dispatch_one_to_all",
           "collect_all_to_all", "dispatch_dp_compute_data_proto", "collect_dp_compute_data_proto",
           "make_nd_compute_dataproto_dispatch_fn", "dispatch_nd_compute", "collect_nd_compute"]

MAGIC_ATTR = "attrs_3141562937"


class _DynamicEnum:
    """Enum-like class whose members can be added at run time."""

    _registry: dict
    _next: int

    def __init__(self, name: str, value: int):
        self.name, self.value = name, value

    def __repr__(self):
        return f"<{type(self).__name__}.{self.name}: {self.value}>"

    def __hash__(self):
        return hash((type(self).__name__, self.name))

    def __eq__(self, other):
        return type(other) is type(self) and other.name == self.name

    @classmethod
    def register(cls, name: str):
        key = name.upper()
        if key not in cls._registry:
            member = cls(key, cls._next)
            cls._registry[key] = member
            setattr(cls, key, member)
            cls._next += 1
        return cls._registry[key]

    @classmethod
    def remove(cls, name: str):
        key = name.upper()
        member = cls._registry.pop(key)
        delattr(cls, key)
        return member

    @classmethod
    def from_name(cls, name: str):
        return cls._registry.get(name.upper())


class Dispatch(_DynamicEnum):
    _registry: dict = {}
    _next = 0


class Execute(_DynamicEnum):
    _registry: dict = {}
    _next = 0


def init_predefined_dispatch_mode():
    for n in ("RANK_ZERO", "ONE_TO_ALL", "ALL_TO_ALL", "DP_COMPUTE", "DP_COMPUTE_PROTO", "DP_COMPUTE_PROTO_WITH_FUNC",
              "DP_COMPUTE_METRIC", "DIRECT_ROLLOUT_METHOD"):
        Dispatch.register(n)
    for n in ("ALL", "RANK_ZERO"):
        Execute.register(n)


init_predefined_dispatch_mode()


# ---------------------------------------------------------------------------------------------- split / merge
_SPLITTABLE = (DataProto, DataProtoFuture, TensorDict)


def _chunk(x, n: int):
    if isinstance(x, TensorDict):
        return chunk_tensordict(x, n)
    return x.chunk(chunks=n)


def _split_args_kwargs(n: int, *args, **kwargs):
    sa = []
    for a in args:
        assert isinstance(a, _SPLITTABLE), f"cannot dispatch argument of type {type(a)} across data-parallel ranks"
        sa.append(_chunk(a, n))
    sk = {}
    for k, v in kwargs.items():
        assert isinstance(v, _SPLITTABLE), f"cannot dispatch kwarg '{k}' of type {type(v)}"
        sk[k] = _chunk(v, n)
    return tuple(sa), sk


def _split_with_auto_padding(n: int, *args, **kwargs):
    """Like ``_split_args_kwargs`` but pads DataProto arguments to a multiple of ``n`` when padding is enabled."""
    from ...protocol import DataProtoConfig, pad_dataproto_to_divisor

    pad = 0
    new_args = []
    for a in args:
        if isinstance(a, DataProto) and a.is_padding_enabled() and len(a) % n:
            a, pad = pad_dataproto_to_divisor(a, n)
        new_args.append(a)
    new_kwargs = {}
    for k, v in kwargs.items():
        if isinstance(v, DataProto) and v.is_padding_enabled() and len(v) % n:
            v, pad = pad_dataproto_to_divisor(v, n)
        new_kwargs[k] = v
    sa, sk = _split_args_kwargs(n, *new_args, **new_kwargs)
    if pad:
        sk[DataProtoConfig.auto_padding_key] = [pad] * n
    return sa, sk


def _concat(outputs: list):
    outputs = [o for o in outputs if o is not None]
    if not outputs:
        return None
    first = outputs[0]
    if isinstance(first, DataProto):
        return DataProto.concat(outputs)
    if isinstance(first, TensorDict):
        return cat_tensordicts(outputs)
    if isinstance(first, DataProtoFuture) or hasattr(first, "result"):
        return DataProtoFuture.concat(outputs)
    raise NotImplementedError(f"cannot collect outputs of type {type(first)}")


# ---------------------------------------------------------------------------------------------- dispatch fns
def dispatch_one_to_all(worker_group, *args, **kwargs):
    n = worker_group.world_size
    return tuple([a] * n for a in args), {k: [v] * n for k, v in kwargs.items()}


def dispatch_all_to_all(worker_group, *args, **kwargs):
    return args, kwargs


def collect_all_to_all(worker_group, output):
    return output


def dispatch_rank_zero(worker_group, *args, **kwargs):
    return tuple([a] for a in args), {k: [v] for k, v in kwargs.items()}


def collect_rank_zero(worker_group, output):
    return output[0]


def dispatch_dp_compute(worker_group, *args, **kwargs):
    n = worker_group.world_size
    for a in list(args) + list(kwargs.values()):
        assert isinstance(a, (tuple, list)) and len(a) == n
    return args, kwargs


def collect_dp_compute(worker_group, output):
    assert len(output) == worker_group.world_size
    return output


def dispatch_dp_compute_data_proto(worker_group, *args, **kwargs):
    return _split_with_auto_padding(worker_group.world_size, *args, **kwargs)


def dispatch_dp_compute_data_proto_with_func(worker_group, *args, **kwargs):
    assert callable(args[0]), "first argument must be the function to run on each shard"
    sa, sk = _split_args_kwargs(worker_group.world_size, *args[1:], **kwargs)
    return ([args[0]] * worker_group.world_size,) + sa, sk


def collect_dp_compute_data_proto(worker_group, output):
    return _concat(collect_dp_compute(worker_group, output))


def collect_dp_compute_metric(worker_group, output):
    """Merge per-rank metric dicts into dict-of-lists."""
    merged: dict[str, list] = {}
    for o in output:
        for k, v in (o or {}).items():
            merged.setdefault(k, []).extend(v if isinstance(v, list) else [v])
    return merged


def dispatch_nd_compute(dp_rank_mapping: list[int], dp_size: int, worker_group, *args, **kwargs):
    """Split into ``dp_size`` chunks and give worker ``i`` chunk ``dp_rank_mapping[i]`` (model-parallel peers of a
    data-parallel rank receive the same chunk)."""
    sa, sk = _split_with_auto_padding(dp_size, *args, **kwargs)
    pick = lambda chunks: [chunks[dp_rank_mapping[i]] for i in range(worker_group.world_size)]
    return tuple(pick(c) for c in sa), {k: (pick(v) if len(v) == dp_size else v) for k, v in sk.items()}


def collect_nd_compute(collect_mask: list[bool], worker_group, output):
    assert len(output) == worker_group.world_size
    return [o for o, keep in zip(output, collect_mask) if keep]


def dispatch_nd_compute_dataproto(dp_rank_mapping, dp_size, worker_group, *args, **kwargs):
    return dispatch_nd_compute(dp_rank_mapping, dp_size, worker_group, *args, **kwargs)


def collect_nd_compute_dataproto(collect_mask, worker_group, output):
    return _concat(collect_nd_compute(collect_mask, worker_group, output))


def dispatch_lazy_compute_data_proto(mesh_name: str, worker_group, *args, **kwargs):
    """Resolve the (dp_rank, is_collect) layout of ``mesh_name`` from the workers on first use, then dispatch."""
    if mesh_name not in worker_group._dispatch_info:
        worker_group._dispatch_info[mesh_name] = worker_group._query_dispatch_info(mesh_name)
    mapping = worker_group._dispatch_info[mesh_name]
    return dispatch_nd_compute_dataproto(mapping, max(mapping) + 1, worker_group, *args, **kwargs)


def collect_lazy_compute_data_proto(mesh_name: str, worker_group, output):
    if mesh_name not in worker_group._collect_info:
        worker_group._collect_info[mesh_name] = worker_group._query_collect_info(mesh_name)
    return collect_nd_compute_dataproto(worker_group._collect_info[mesh_name], worker_group, output)


def make_nd_compute_dataproto_dispatch_fn(mesh_name: str) -> dict:
    return {"dispatch_fn": partial(dispatch_lazy_compute_data_proto, mesh_name),
            "collect_fn": partial(collect_lazy_compute_data_proto, mesh_name)}


def dummy_direct_rollout_call(worker_group, *args, **kwargs):
    raise NotImplementedError("Direct rollout call is forbidden.")


DISPATCH_MODE_FN_REGISTRY: dict = {
    Dispatch.ONE_TO_ALL: {"dispatch_fn": dispatch_one_to_all, "collect_fn": collect_all_to_all},
    Dispatch.ALL_TO_ALL: {"dispatch_fn": dispatch_all_to_all, "collect_fn": collect_all_to_all},
    Dispatch.RANK_ZERO: {"dispatch_fn": dispatch_rank_zero, "collect_fn": collect_rank_zero},
    Dispatch.DP_COMPUTE: {"dispatch_fn": dispatch_dp_compute, "collect_fn": collect_dp_compute},
    Dispatch.DP_COMPUTE_PROTO: {"dispatch_fn": dispatch_dp_compute_data_proto, "collect_fn": collect_dp_compute_data_proto},
    Dispatch.DP_COMPUTE_PROTO_WITH_FUNC: {"dispatch_fn": dispatch_dp_compute_data_proto_with_func,
                                          "collect_fn": collect_dp_compute_data_proto},
    Dispatch.DP_COMPUTE_METRIC: {"dispatch_fn": dispatch_dp_compute_data_proto, "collect_fn": collect_dp_compute_metric},
    Dispatch.DIRECT_ROLLOUT_METHOD: {"dispatch_fn": dummy_direct_rollout_call, "collect_fn": dummy_direct_rollout_call},
}


def get_predefined_dispatch_fn(dispatch_mode):
    return DISPATCH_MODE_FN_REGISTRY[dispatch_mode]


def register_dispatch_mode(dispatch_mode_name: str, dispatch_fn: Callable, collect_fn: Callable):
    mode = Dispatch.register(dispatch_mode_name)
    assert mode not in DISPATCH_MODE_FN_REGISTRY, f"dispatch_mode_name {dispatch_mode_name} already exists"
    DISPATCH_MODE_FN_REGISTRY[mode] = {"dispatch_fn": dispatch_fn, "collect_fn": collect_fn}
    return mode


def update_dispatch_mode(dispatch_mode, dispatch_fn: Callable, collect_fn: Callable):
    assert dispatch_mode in DISPATCH_MODE_FN_REGISTRY
    DISPATCH_MODE_FN_REGISTRY[dispatch_mode] = {"dispatch_fn": dispatch_fn, "collect_fn": collect_fn}


def get_predefined_execute_fn(execute_mode):
    return {Execute.ALL: {"execute_fn_name": "execute_all"}, Execute.RANK_ZERO: {"execute_fn_name": "execute_rank_zero"}}[execute_mode]


def _check_dispatch_mode(dispatch_mode):
    assert isinstance(dispatch_mode, (Dispatch, dict)), f"dispatch_mode must be a Dispatch or a Dict. Got {dispatch_mode}"
    if isinstance(dispatch_mode, dict):
        for key in ("dispatch_fn", "collect_fn"):
            assert key in dispatch_mode, f"key {key} should be in dispatch_mode if it is a dictionary"


def _materialize_futures(*args, **kwargs):
    args = tuple(a.get() if isinstance(a, DataProtoFuture) else a for a in args)
    kwargs = {k: (v.get() if isinstance(v, DataProtoFuture) else v) for k, v in kwargs.items()}
    return args, kwargs


def register(dispatch_mode=Dispatch.ALL_TO_ALL, execute_mode=Execute.ALL, blocking: bool = True,
             materialize_futures: bool = True):
    """Mark a worker method as remotely callable through its worker group."""
    _check_dispatch_mode(dispatch_mode)
    assert isinstance(execute_mode, Execute)

    def decorator(func):
        if inspect.iscoroutinefunction(func):
            @wraps(func)
            async def inner(*args, **kwargs):
                if materialize_futures:
                    args, kwargs = _materialize_futures(*args, **kwargs)
                return await func(*args, **kwargs)
        else:
            @wraps(func)
            def inner(*args, **kwargs):
                if materialize_futures:
                    args, kwargs = _materialize_futures(*args, **kwargs)
                return func(*args, **kwargs)

        setattr(inner, MAGIC_ATTR, {"dispatch_mode": dispatch_mode, "execute_mode": execute_mode, "blocking": blocking})
        return inner

    return decorator
