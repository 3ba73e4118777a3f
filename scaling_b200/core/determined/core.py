"""Glue for running under the Determined cluster manager (src/scaling/core/determined/core.py:6-19,
src/scaling/core/utils/determined_utils.py:19-44).

``determined`` is an optional dependency: everything here imports without it, and only the functions that need the
package raise when it is missing.
"""

from __future__ import annotations

import contextlib
import faulthandler
from typing import Any, Iterator

try:  # pragma: no cover - depends on the installation
    import determined as det

    DETERMINED_AVAILABLE = True
except ImportError:  # pragma: no cover
    det = None
    DETERMINED_AVAILABLE = False


def _require() -> Any:
    if det is None:
        raise ImportError("the `determined` package is not installed; install it to run under a Determined master")
    return det


def init(*args: Any, **kwargs: Any) -> Any:
    """``det.core.init`` with tensorboard files flushed manually (the automatic mode writes far too many files for
    shared file systems); callers may not override that."""
    assert "tensorboard_mode" not in kwargs, "We don't allow any overwrite for tensorboard_mode"
    d = _require()
    kwargs = dict(kwargs)
    kwargs["tensorboard_mode"] = d.core._tensorboard_mode.TensorboardMode.MANUAL
    return d.core.init(*args, **kwargs)


@contextlib.contextmanager
def maybe_periodic_stacktraces(debug_enabled: bool, every_seconds: int = 30) -> Iterator[None]:
    """With ``debug_enabled``: dump every thread's stack to stderr every ``every_seconds`` while the block runs."""
    if debug_enabled:
        faulthandler.dump_traceback_later(every_seconds, repeat=True)
    try:
        yield
    finally:
        if debug_enabled:
            faulthandler.cancel_dump_traceback_later()


def determined_profiler_from_ctx(ctx: Any, config_determined: Any, info: Any) -> Any:
    """Determined's system-metrics profiler agent for this trial and rank."""
    d = _require()
    import determined.profiler  # noqa: F401

    begin_on_batch, end_after_batch = config_determined.profiling_interval()
    return d.profiler.ProfilerAgent(
        trial_id=str(ctx.train._trial_id), agent_id=info.agent_id, master_url=info.master_url,
        profiling_is_enabled=config_determined.profiling_enabled(), global_rank=ctx.distributed.get_rank(),
        local_rank=ctx.distributed.get_local_rank(), begin_on_batch=begin_on_batch, end_after_batch=end_after_batch,
        sync_timings=config_determined.profiling_sync_timings(),
    )
