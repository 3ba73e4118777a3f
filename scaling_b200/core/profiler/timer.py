"""Timers for the step loop.

``SynchronizedTimer`` keeps the reference's semantics (wall clock between two device
synchronisations, src/scaling/core/profiler/timer.py:7-35).  ``CudaEventTimer`` is the
B200-native replacement used inside the instruction loop: it records CUDA events on the launching
stream and is read after the step, so profiling does not serialise the device.
"""

from __future__ import annotations

import time
from typing import Optional

import torch


def _sync() -> None:
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        torch.cuda.synchronize()


class SynchronizedTimer:
    def __init__(self) -> None:
        self._start: Optional[float] = None
        self._stop: Optional[float] = None

    def start(self) -> None:
        _sync()
        self._start = time.time()

    def stop(self) -> None:
        _sync()
        self._stop = time.time()

    def reset(self) -> None:
        self._start = self._stop = None

    def duration(self) -> float:
        assert self._start is not None and self._stop is not None, "timer was not started and stopped"
        return self._stop - self._start


class CudaEventTimer:
    """Device-side duration between two points of the current stream (host clock on CPU ranks)."""

    def __init__(self) -> None:
        self._cuda = torch.cuda.is_available()
        self._e0 = self._e1 = None
        self._t0 = self._t1 = 0.0

    def start(self) -> None:
        if self._cuda:
            self._e0 = torch.cuda.Event(enable_timing=True)
            self._e1 = torch.cuda.Event(enable_timing=True)
            self._e0.record()
        else:
            self._t0 = time.perf_counter()

    def stop(self) -> None:
        if self._cuda:
            self._e1.record()
        else:
            self._t1 = time.perf_counter()

    def duration(self) -> float:
        """Seconds; synchronises on the stop event only."""
        if self._cuda:
            self._e1.synchronize()
            return self._e0.elapsed_time(self._e1) / 1000.0
        return self._t1 - self._t0
