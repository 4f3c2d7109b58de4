"""Process-group bootstrap. One process per GPU; NCCL for device tensors, gloo for host tensors.

Parity target: ``verl/utils/distributed.py`` (``initialize_global_process_group_ray`` :82-98 with backend
``cpu:gloo,cuda:nccl`` and the ``nccl_timeout``; ``set_numa_affinity`` :30; ``stateless_init_process_group`` :124).
"""

from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist

from .device import get_device_name

__all__ = ["initialize_global_process_group", "initialize_global_process_group_ray", "destroy_global_process_group",
           "set_numa_affinity", "stateless_init_process_group", "get_world_size", "get_rank", "set_data_parallel_group",
           "get_data_parallel_group"]

_DP_GROUP = None


def set_data_parallel_group(group) -> None:
    """Restrict the training engines created afterwards to ``group`` (e.g. the trainer ranks of a job whose other
    ranks only serve rollout). ``None`` restores the default: all ranks."""
    global _DP_GROUP
    _DP_GROUP = group


def get_data_parallel_group():
    return _DP_GROUP


def initialize_global_process_group(timeout_second: int = 600, spmd: bool = False):
    """Idempotent init from WORLD_SIZE/RANK/MASTER_* env; single-process runs skip the process group."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if get_device_name() == "cuda":
        torch.cuda.set_device(local_rank % max(1, torch.cuda.device_count()))
    if world > 1 and not dist.is_initialized():
        backend = "cpu:gloo,cuda:nccl" if get_device_name() == "cuda" else "gloo"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = {}
        if get_device_name() == "cuda":
            kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_second), **kw)
    return local_rank, rank, world


initialize_global_process_group_ray = initialize_global_process_group


def destroy_global_process_group() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def get_rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def set_numa_affinity() -> None:
    """Bind the process to the CPUs of the NUMA node nearest to its GPU (best effort; needs NVML)."""
    if get_device_name() != "cuda":
        return
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
        n = os.cpu_count() or 1
        words = (n + 63) // 64
        aff = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = [i for i in range(n) if (aff[i // 64] >> (i % 64)) & 1]
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception:
        pass


def stateless_init_process_group(master_address: str, master_port: int, rank: int, world_size: int, device=None):
    """A process group that does not touch the global default group (used for trainer <-> rollout weight links)."""
    store = dist.TCPStore(master_address, int(master_port), world_size, is_master=(rank == 0),
                          timeout=datetime.timedelta(seconds=300))
    backend = "nccl" if (device is not None and torch.device(device).type == "cuda") else "gloo"
    opts = {}
    pg = dist.distributed_c10d._new_process_group_helper(  # type: ignore[attr-defined]
        world_size, rank, [], backend, store, group_name=f"stateless_{master_port}",
        timeout=datetime.timedelta(seconds=300), **opts) if hasattr(dist.distributed_c10d, "_new_process_group_helper") else None
    return pg
