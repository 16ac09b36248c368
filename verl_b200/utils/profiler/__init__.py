from .config import ProfilerConfig  # noqa: F401
from .performance import GPUMemoryLogger, DeviceTimer, log_gpu_memory_usage, reduce_timing, simple_timer, marked_timer  # noqa: F401
from .profile import DistProfiler, DistProfilerExtension  # noqa: F401
