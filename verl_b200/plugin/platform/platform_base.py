"""The questions a device platform answers. One subclass per kind of accelerator; the framework itself ships the B200
(CUDA, sm_100a) platform and a CPU platform that serves as the numerical oracle in tests."""

from __future__ import annotations

import abc
import shutil
import subprocess
from contextlib import contextmanager
from types import ModuleType
from typing import Any, Optional

__all__ = ["PlatformBase"]


class PlatformBase(abc.ABC):
    # ---- identity
    @property
    @abc.abstractmethod
    def device_name(self) -> str:
        """Device type string for ``torch.device`` ("cuda", "cpu", ...)."""

    @property
    @abc.abstractmethod
    def vendor_name(self) -> str: ...

    @property
    @abc.abstractmethod
    def device_module(self) -> ModuleType:
        """The ``torch.<device>`` module."""

    @abc.abstractmethod
    def is_available(self) -> bool: ...

    @staticmethod
    def check_smi_command(cmd: str) -> bool:
        """True when the vendor's management tool exists and exits 0 (a read-only query)."""
        exe = shutil.which(cmd.split()[0])
        if exe is None:
            return False
        try:
            return subprocess.run(cmd.split(), stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, timeout=10).returncode == 0
        except Exception:
            return False

    def is_platform_available(self, use_smi_check: bool = False) -> bool:
        return self.is_available() and (not use_smi_check or self.check_smi_command(self.smi_command()))

    def smi_command(self) -> str:
        return "true"

    # ---- devices
    @abc.abstractmethod
    def current_device(self) -> int: ...

    @abc.abstractmethod
    def device_count(self) -> int: ...

    @abc.abstractmethod
    def set_device(self, device_index: int) -> None: ...

    @abc.abstractmethod
    def synchronize(self, device_index: Optional[int] = None) -> None: ...

    @abc.abstractmethod
    def manual_seed(self, seed: int) -> None: ...

    @abc.abstractmethod
    def manual_seed_all(self, seed: int) -> None: ...

    @abc.abstractmethod
    def set_allocator_settings(self, settings: str) -> None: ...

    @abc.abstractmethod
    def empty_cache(self) -> None: ...

    @abc.abstractmethod
    def get_device_capability(self, device_index: int = 0) -> tuple[Optional[int], Optional[int]]: ...

    def get_device_uuid(self, device_id: int) -> str:
        return f"{self.device_name}:{device_id}"

    # ---- communication and process placement
    @abc.abstractmethod
    def communication_backend_name(self) -> str:
        """``torch.distributed`` backend for device tensors."""

    @abc.abstractmethod
    def visible_devices_envvar(self) -> str: ...

    @abc.abstractmethod
    def is_ipc_supported(self) -> bool:
        """Whether device memory can be shared between processes / mapped by peers."""

    def get_collective_module(self) -> Any:
        import torch.distributed as dist

        return dist

    @abc.abstractmethod
    def ray_resource_name(self) -> str: ...

    @abc.abstractmethod
    def ray_noset_envvars(self) -> list[str]:
        """Variables that stop Ray from rewriting the visible-devices variable of its workers."""

    def ray_resource_options(self, num_gpus: float) -> dict[str, Any]:
        name = self.ray_resource_name()
        return {"num_gpus": num_gpus} if name == "GPU" else {"resources": {name: num_gpus}}

    def rollout_env_vars(self) -> dict[str, str]:
        """Extra environment for rollout server processes."""
        return {}

    # ---- profiling
    @abc.abstractmethod
    @contextmanager
    def nvtx_range(self, msg: str):
        yield

    @abc.abstractmethod
    def profiler_start(self) -> None: ...

    @abc.abstractmethod
    def profiler_stop(self) -> None: ...

    @abc.abstractmethod
    def cudart(self) -> Any:
        """Runtime handle for profiler control, or None."""

    # ---- models
    def apply_model_patches(self, model_type: str) -> None:
        """Hook for platforms that replace library kernels of a model family. This framework's own decoder needs none."""
        return None

    def default_dtype(self):
        import torch

        return torch.bfloat16 if self.device_name != "cpu" else torch.float32
