from .base import InProcessWorkerGroup, MultiprocessWorkerGroup, SPMDWorkerGroup  # noqa: F401
