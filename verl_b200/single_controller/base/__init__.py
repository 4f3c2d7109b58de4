from .decorator import Dispatch, Execute, register, make_nd_compute_dataproto_dispatch_fn  # noqa: F401
from .worker import Worker  # noqa: F401
from .worker_group import ClassWithInitArgs, ResourcePool, WorkerGroup  # noqa: F401
