"""Device helpers (the framework targets NVIDIA B200; CPU is the test/oracle device).

Parity target: ``verl/utils/device.py`` and ``verl/plugin/platform/platform_base.py``.
"""

from __future__ import annotations

import os

import torch

__all__ = ["is_cuda_available", "get_device_name", "get_torch_device", "get_device_id", "get_nccl_backend",
           "get_visible_devices_keyword", "is_support_ipc", "get_device_capability", "set_expandable_segments",
           "auto_set_device", "get_default_dtype"]

is_cuda_available = torch.cuda.is_available()


def get_device_name() -> str:
    forced = os.getenv("VERL_ENGINE_DEVICE")
    if forced:
        return forced
    return "cuda" if torch.cuda.is_available() else "cpu"


def _platform():
    """The active device platform (``verl_b200.plugin.platform``); the helpers below are its short forms."""
    from ..plugin.platform import get_platform

    p = get_platform()
    if p.device_name != get_device_name() and not os.getenv("VERL_PLATFORM"):
        # the device was forced after the platform was first detected (tests switch to the CPU oracle): detect again
        from ..plugin.platform import set_platform

        set_platform(None)
        p = get_platform()
    return p


def get_torch_device():
    return _platform().device_module


def get_device_id() -> int:
    return _platform().current_device()


def get_nccl_backend() -> str:
    return _platform().communication_backend_name()


def get_visible_devices_keyword() -> str:
    return _platform().visible_devices_envvar()


def is_support_ipc() -> bool:
    return _platform().is_ipc_supported()


def get_device_capability(device_id: int = 0):
    return _platform().get_device_capability(device_id)


def set_expandable_segments(enable: bool) -> None:
    if get_device_name() == "cuda" and hasattr(torch.cuda.memory, "_set_allocator_settings"):
        torch.cuda.memory._set_allocator_settings(f"expandable_segments:{enable}")


def auto_set_device(config) -> None:
    """Point every ``device`` entry of a trainer config at the device this process actually has."""
    dev = get_device_name()
    try:
        if config.trainer.get("device", dev) != dev:
            config.trainer.device = dev
    except Exception:
        pass


def get_default_dtype() -> torch.dtype:
    return torch.bfloat16 if get_device_name() == "cuda" else torch.float32
