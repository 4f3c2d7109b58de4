"""Host CPU: the oracle platform (fp32, gloo) on which every path of the framework also runs."""

from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Optional

import torch

from .platform_base import PlatformBase
from .platform_manager import PlatformRegistry

__all__ = ["PlatformCPU"]


@PlatformRegistry.register("cpu")
class PlatformCPU(PlatformBase):
    device_name = "cpu"
    vendor_name = "host"

    @property
    def device_module(self):
        return torch.cpu

    def is_available(self) -> bool:
        return True

    def current_device(self) -> int:
        return 0

    def device_count(self) -> int:
        return 1

    def set_device(self, device_index: int) -> None:
        return None

    def synchronize(self, device_index: Optional[int] = None) -> None:
        return None

    def manual_seed(self, seed: int) -> None:
        torch.manual_seed(seed)

    def manual_seed_all(self, seed: int) -> None:
        torch.manual_seed(seed)

    def set_allocator_settings(self, settings: str) -> None:
        return None

    def empty_cache(self) -> None:
        return None

    def get_device_capability(self, device_index: int = 0):
        return (None, None)

    def communication_backend_name(self) -> str:
        return "gloo"

    def visible_devices_envvar(self) -> str:
        return "CUDA_VISIBLE_DEVICES"

    def is_ipc_supported(self) -> bool:
        return False

    def ray_resource_name(self) -> str:
        return "CPU"

    def ray_noset_envvars(self) -> list[str]:
        return []

    def ray_resource_options(self, num_gpus: float) -> dict[str, Any]:
        return {"num_cpus": max(1, int(num_gpus))}

    @contextmanager
    def nvtx_range(self, msg: str):
        yield

    def profiler_start(self) -> None:
        return None

    def profiler_stop(self) -> None:
        return None

    def cudart(self) -> Any:
        return None
