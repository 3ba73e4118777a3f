from .core import DETERMINED_AVAILABLE, determined_profiler_from_ctx, init, maybe_periodic_stacktraces

__all__ = ["DETERMINED_AVAILABLE", "determined_profiler_from_ctx", "init", "maybe_periodic_stacktraces"]
