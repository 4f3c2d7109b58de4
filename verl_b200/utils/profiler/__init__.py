from .performance import GPUMemoryLogger, log_gpu_memory_usage, marked_timer, reduce_timing, gather_timing, simple_timer  # noqa: F401
from .profile import DistProfiler, DistProfilerExtension, ProfilerConfig, mark_start_range, mark_end_range, mark_annotate  # noqa: F401
