"""Registry and selection of the active device platform."""

from __future__ import annotations

import os
from typing import Optional

from .platform_base import PlatformBase

__all__ = ["PlatformRegistry", "get_platform", "set_platform"]


class PlatformRegistry:
    """name -> platform class. Out-of-tree platforms register under their own name before ``get_platform`` is first called
    (import them from ``VERL_PLATFORM_MODULE``) and are selected with ``VERL_PLATFORM``."""

    _platforms: dict[str, type[PlatformBase]] = {}

    @classmethod
    def register(cls, platform: str):
        def decorator(platform_cls: type[PlatformBase]) -> type[PlatformBase]:
            assert issubclass(platform_cls, PlatformBase), f"{platform_cls.__name__} must be a subclass of PlatformBase"
            cls._platforms[platform.lower()] = platform_cls
            return platform_cls

        return decorator

    @classmethod
    def get(cls, name: str) -> Optional[type[PlatformBase]]:
        return cls._platforms.get(name.lower())

    @classmethod
    def registered_names(cls) -> tuple[str, ...]:
        return tuple(sorted(cls._platforms))


_ACTIVE: Optional[PlatformBase] = None


def _detect_platform_name() -> str:
    forced = os.environ.get("VERL_PLATFORM")
    if forced:
        return forced.lower()
    from ...utils.device import get_device_name

    return "b200" if get_device_name() == "cuda" else "cpu"


def _create_platform(name: str) -> PlatformBase:
    from . import platform_b200, platform_cpu  # noqa: F401  (self-registering)

    extra = os.environ.get("VERL_PLATFORM_MODULE")
    if extra:
        import importlib

        importlib.import_module(extra)
    cls = PlatformRegistry.get(name)
    if cls is None:
        raise ValueError(f"unknown platform {name!r}; registered: {PlatformRegistry.registered_names()}")
    return cls()


def get_platform() -> PlatformBase:
    global _ACTIVE
    if _ACTIVE is None:
        _ACTIVE = _create_platform(_detect_platform_name())
    return _ACTIVE


def set_platform(platform: Optional[PlatformBase]) -> None:
    """Install a platform instance (None: detect again on the next ``get_platform``)."""
    global _ACTIVE
    assert platform is None or isinstance(platform, PlatformBase)
    _ACTIVE = platform
