from .profiler import Profiler, ProfilerObservation
from .profiler_config import ProfilerConfig
from .timer import CudaEventTimer, SynchronizedTimer

__all__ = ["CudaEventTimer", "Profiler", "ProfilerConfig", "ProfilerObservation", "SynchronizedTimer"]
