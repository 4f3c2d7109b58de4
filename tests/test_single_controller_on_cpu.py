"""Dispatch / collect semantics on an in-process fake cluster and a real multi-process gloo group."""
import numpy as np
import pytest
import torch

from verl_b200 import DataProto
from verl_b200.single_controller.base import ClassWithInitArgs, Dispatch, Execute, Worker, register
from verl_b200.single_controller.base.decorator import make_nd_compute_dataproto_dispatch_fn, register_dispatch_mode
from verl_b200.single_controller.local import InProcessWorkerGroup, MultiprocessWorkerGroup


class Toy(Worker):
    def __init__(self, k):
        super().__init__()
        self.k = k
        self._register_dispatch_collect_info("mesh", dp_rank=self.rank // 2, is_collect=self.rank % 2 == 0)

    @register(Dispatch.ONE_TO_ALL)
    def scale(self, x):
        return x * self.k + self.rank

    @register(Dispatch.DP_COMPUTE_PROTO)
    def per_rank(self, d):
        return DataProto.from_dict({"y": d.batch["x"] * 10 + self.rank})

    @register(Dispatch.ALL_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def only_zero(self, x):
        return (self.rank, x)

    @register(make_nd_compute_dataproto_dispatch_fn("mesh"))
    def nd(self, d):
        return DataProto.from_dict({"y": d.batch["x"] + 100 * self.rank})

    @register(Dispatch.DP_COMPUTE_METRIC)
    def metric(self, d):
        return {"n": [len(d)], "rank": self.rank}

    @register(Dispatch.ONE_TO_ALL)
    def boom(self):
        if self.rank == 1:
            raise ValueError("injected failure on rank 1")
        return "fine"

    @register(Dispatch.ONE_TO_ALL)
    def allreduce(self):
        import torch.distributed as dist

        from verl_b200.utils.distributed import initialize_global_process_group

        initialize_global_process_group()
        t = torch.tensor([float(self.rank + 1)])
        dist.all_reduce(t)
        return t.item()


def test_inprocess_dispatch_modes():
    wg = InProcessWorkerGroup(4, ClassWithInitArgs(Toy, 2))
    assert wg.world_size == 4 and wg.scale(3) == [6, 7, 8, 9]
    d = DataProto.from_dict({"x": torch.arange(8)})
    assert wg.per_rank(d).batch["y"].tolist() == [0, 10, 21, 31, 42, 52, 63, 73]
    assert wg.only_zero("a") == (0, "a")
    # 2 dp ranks x 2 model-parallel peers: peers get the same chunk, only even ranks are collected
    assert wg.nd(d).batch["y"].tolist() == [0, 1, 2, 3, 204, 205, 206, 207]
    m = wg.metric(d)
    assert m["n"] == [2, 2, 2, 2] and m["rank"] == [0, 1, 2, 3]


def test_auto_padding_roundtrip(monkeypatch):
    wg = InProcessWorkerGroup(4, ClassWithInitArgs(Toy, 1))
    d = DataProto.from_dict({"x": torch.arange(6)}, auto_padding=True)
    out = wg.per_rank(d)
    assert len(out) == 6 and (out.batch["y"] // 10).tolist() == list(range(6))


def test_custom_dispatch_mode():
    mode = register_dispatch_mode("REVERSED_TEST", lambda wg, x: (([x] * wg.world_size,), {}), lambda wg, out: out[::-1])

    class W2(Worker):
        @register(mode)
        def f(self, x):
            return self.rank + x

    assert InProcessWorkerGroup(3, ClassWithInitArgs(W2)).f(10) == [12, 11, 10]


def test_multiprocess_group_gloo_and_failure_detection():
    wg = MultiprocessWorkerGroup(2, ClassWithInitArgs(Toy, 3), device="cpu", start_timeout=120)
    try:
        assert wg.scale(1) == [3, 4]
        assert wg.allreduce() == [3.0, 3.0]
        assert all(wg._is_worker_alive(w) for w in wg._workers)
        # a worker whose method raises surfaces as a driver-side error naming the rank
        with pytest.raises(RuntimeError, match="worker 1 failed in 'boom'"):
            wg.boom()
        assert wg.scale(2) == [6, 7]  # the group stays usable after a host-side failure
    finally:
        wg.shutdown()
    assert not any(p.is_alive() for p in wg._procs)


class _Adder(Worker):
    def __init__(self, bias):
        super().__init__()
        self.bias = bias
        self._register_dispatch_collect_info("adder", dp_rank=self.rank, is_collect=True)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def add(self, x):
        return x + self.bias + 100 * self.rank

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn(mesh_name="adder"))
    def add_rows(self, data):
        return DataProto.from_dict(tensors={"y": data.batch["x"] + self.bias})


class _Scaler(Worker):
    def __init__(self, factor):
        super().__init__()
        self.factor = factor

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def scale(self, x):
        # the roles of a fused worker see each other
        return x * self.factor + self.fused_worker_dict["adder"].bias


@pytest.mark.parametrize("backend", ["inprocess", "multiprocess"])
def test_fused_worker_roles_share_processes(backend):
    from verl_b200.single_controller.base.fused import create_colocated_worker_cls_fused
    from verl_b200.single_controller.local import InProcessWorkerGroup, MultiprocessWorkerGroup

    cia = create_colocated_worker_cls_fused({"adder": ClassWithInitArgs(_Adder, bias=7), "scaler": ClassWithInitArgs(_Scaler, factor=3)})
    assert cia.cls.__name__ == "FusedWorker_adder_scaler" and cia.cls.is_fused_worker
    wg = (InProcessWorkerGroup if backend == "inprocess" else MultiprocessWorkerGroup)(2, cia)
    views = wg.spawn_fused({"adder", "scaler"})
    assert views["adder"].add(1) == [8, 108] and views["scaler"].scale(2) == [13, 13]
    assert not hasattr(views["adder"], "scale") and views["adder"].world_size == 2
    out = views["adder"].add_rows(DataProto.from_dict(tensors={"x": torch.arange(4.0)}))   # nd-mesh dispatch through the view
    assert torch.equal(out.batch["y"], torch.arange(4.0) + 7)
    wg.fuse({"adder", "scaler"})
    assert wg.adder.add(0) == [7, 107] and wg.scaler.scale(1) == [10, 10]
    if hasattr(wg, "shutdown"):
        wg.shutdown()
