"""Device platform interface: what the rest of the framework asks of the accelerator it runs on.

``get_platform()`` returns the active platform: :class:`PlatformB200` on a machine with CUDA devices, the CPU oracle
platform otherwise. An out-of-tree platform registers itself with ``@PlatformRegistry.register("name")`` and is chosen by
``VERL_PLATFORM=name`` (or installed with ``set_platform``).

Parity target: ``verl/plugin/platform/platform_base.py:20-268``, ``platform_manager.py``.
"""

from .platform_base import PlatformBase
from .platform_manager import PlatformRegistry, get_platform, set_platform

__all__ = ["PlatformBase", "PlatformRegistry", "get_platform", "set_platform"]
