"""NVIDIA B200 (CUDA, sm_100a): the platform this framework is written for."""

from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Optional

import torch

from .platform_base import PlatformBase
from .platform_manager import PlatformRegistry

__all__ = ["PlatformB200"]


@PlatformRegistry.register("cuda")
@PlatformRegistry.register("b200")
class PlatformB200(PlatformBase):
    device_name = "cuda"
    vendor_name = "nvidia"

    @property
    def device_module(self):
        return torch.cuda

    def is_available(self) -> bool:
        return torch.cuda.is_available()

    def smi_command(self) -> str:
        return "nvidia-smi -L"

    def current_device(self) -> int:
        return torch.cuda.current_device()

    def device_count(self) -> int:
        return torch.cuda.device_count()

    def set_device(self, device_index: int) -> None:
        torch.cuda.set_device(device_index)

    def synchronize(self, device_index: Optional[int] = None) -> None:
        torch.cuda.synchronize(device_index)

    def manual_seed(self, seed: int) -> None:
        torch.cuda.manual_seed(seed)

    def manual_seed_all(self, seed: int) -> None:
        torch.cuda.manual_seed_all(seed)

    def set_allocator_settings(self, settings: str) -> None:
        torch.cuda.memory._set_allocator_settings(settings)

    def empty_cache(self) -> None:
        torch.cuda.empty_cache()

    def get_device_capability(self, device_index: int = 0):
        return torch.cuda.get_device_capability(device_index) if self.is_available() else (None, None)

    def get_device_uuid(self, device_id: int) -> str:
        return str(torch.cuda.get_device_properties(device_id).uuid)

    def communication_backend_name(self) -> str:
        return "nccl"

    def visible_devices_envvar(self) -> str:
        return "CUDA_VISIBLE_DEVICES"

    def is_ipc_supported(self) -> bool:
        return True

    def ray_resource_name(self) -> str:
        return "GPU"

    def ray_noset_envvars(self) -> list[str]:
        return ["RAY_EXPERIMENTAL_NOSET_CUDA_VISIBLE_DEVICES"]

    def rollout_env_vars(self) -> dict[str, str]:
        return {"NCCL_CUMEM_ENABLE": "0"}

    @contextmanager
    def nvtx_range(self, msg: str):
        torch.cuda.nvtx.range_push(msg)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()

    def profiler_start(self) -> None:
        torch.cuda.cudart().cudaProfilerStart()

    def profiler_stop(self) -> None:
        torch.cuda.cudart().cudaProfilerStop()

    def cudart(self) -> Any:
        return torch.cuda.cudart()
