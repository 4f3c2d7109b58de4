"""Base class of everything that runs on a device rank under a worker group.

Parity target: ``verl/single_controller/base/worker.py`` (env-driven rank discovery :181-220, dispatch-mesh
registration :86-118, helper executors :320-348).
"""

from __future__ import annotations

import os
import socket
from dataclasses import dataclass

from .decorator import Dispatch, Execute, register

__all__ = ["Worker", "DistRankInfo", "DistGlobalInfo", "WorkerHelper"]


@dataclass
class DistRankInfo:
    tp_rank: int
    dp_rank: int
    pp_rank: int
    cp_rank: int = 0


@dataclass
class DistGlobalInfo:
    tp_size: int
    dp_size: int
    pp_size: int
    cp_size: int = 1


class WorkerHelper:
    @staticmethod
    def _get_node_ip() -> str:
        try:
            return socket.gethostbyname(socket.gethostname())
        except Exception:
            return "127.0.0.1"

    @staticmethod
    def _get_free_port() -> int:
        with socket.socket() as s:
            s.bind(("", 0))
            return s.getsockname()[1]

    def get_availale_master_addr_port(self):
        return self._get_node_ip(), str(self._get_free_port())

    get_available_master_addr_port = get_availale_master_addr_port


class Worker(WorkerHelper):
    """Reads its coordinates (WORLD_SIZE, RANK, LOCAL_RANK, MASTER_ADDR/PORT) from the environment."""

    fused_worker_attr_name = "fused_worker_dict"

    def __init__(self, cuda_visible_devices=None) -> None:
        self._world_size = int(os.environ.get("WORLD_SIZE", 1))
        self._rank = int(os.environ.get("RANK", 0))
        self._local_rank = int(os.environ.get("LOCAL_RANK", 0))
        self._local_world_size = int(os.environ.get("LOCAL_WORLD_SIZE", self._world_size))
        self._master_addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        self._master_port = os.environ.get("MASTER_PORT", "29500")
        self._dispatch_mesh: dict[str, tuple[int, bool]] = {}
        self.fused_worker_dict = {}

    # -- dispatch-mesh registry (which data-parallel chunk this worker consumes; whether its output is collected)
    def _register_dispatch_collect_info(self, mesh_name: str, dp_rank: int, is_collect: bool) -> None:
        if mesh_name in self._dispatch_mesh:
            raise ValueError(f"mesh_name {mesh_name} has been registered")
        self._dispatch_mesh[mesh_name] = (int(dp_rank), bool(is_collect))

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def _query_dispatch_info(self, mesh_name: str) -> int:
        assert mesh_name in self._dispatch_mesh, f"{mesh_name} is not registered in {type(self).__name__}"
        return self._dispatch_mesh[mesh_name][0]

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def _query_collect_info(self, mesh_name: str) -> bool:
        assert mesh_name in self._dispatch_mesh, f"{mesh_name} is not registered in {type(self).__name__}"
        return self._dispatch_mesh[mesh_name][1]

    # -- info
    @property
    def world_size(self) -> int:
        return self._world_size

    @property
    def rank(self) -> int:
        return self._rank

    def get_master_addr_port(self):
        return self._master_addr, self._master_port

    def get_cuda_visible_devices(self):
        return os.environ.get("CUDA_VISIBLE_DEVICES", "not set")

    # -- generic executors
    @register(dispatch_mode=Dispatch.DP_COMPUTE_PROTO_WITH_FUNC)
    def execute_with_func_generator(self, func, *args, **kwargs):
        return func(self, *args, **kwargs)

    @register(dispatch_mode=Dispatch.ALL_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def execute_func_rank_zero(self, func, *args, **kwargs):
        return func(*args, **kwargs)
