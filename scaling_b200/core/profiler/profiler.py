"""Per-instruction profiler of the pipeline engine.

Observations have the reference's record layout (timer name, step, micro batch, buffer, pipe/data/
model coordinates, duration; src/scaling/core/profiler/profiler.py:13-139) and are gathered to rank
0 into one json file that the schedule visualiser can replay.  Durations come from CUDA events that
are read when the step is flushed, not from device-wide synchronisations around every instruction.
"""

from __future__ import annotations

import contextlib
import json
from pathlib import Path
from typing import Iterator, NamedTuple, Optional

import torch.distributed as dist

from ...parallel.topology import Topology
from .profiler_config import ProfilerConfig
from .timer import CudaEventTimer


class ProfilerObservation(NamedTuple):
    timer_name: str
    step: int
    micro_batch_id: Optional[int]
    buffer_id: Optional[int]
    pipe_parallel_rank: int
    data_parallel_rank: int
    model_parallel_rank: int
    duration: float


class Profiler:
    def __init__(self, config: ProfilerConfig, topology: Topology) -> None:
        self.config = config
        self.topology = topology
        self.current_step = 0
        self._open: dict[tuple, CudaEventTimer] = {}
        self._pending: list[tuple[str, int, Optional[int], Optional[int], CudaEventTimer]] = []
        self.observations: list[ProfilerObservation] = []
        self._saved = False

    @property
    def active(self) -> bool:
        c = self.config
        return c.profile_steps > 0 and c.profile_start_at_step <= self.current_step < c.profile_start_at_step + c.profile_steps

    def step(self) -> None:
        self.current_step += 1

    def flush(self) -> None:
        """Resolve event timers of the finished step; save once the profiling window has passed."""
        t = self.topology
        for name, step, mb, buf, timer in self._pending:
            self.observations.append(
                ProfilerObservation(name, step, mb, buf, t.pipe_parallel_rank, t.data_parallel_rank,
                                    t.model_parallel_rank, timer.duration())
            )
        self._pending.clear()
        c = self.config
        if c.profile_steps > 0 and not self._saved and self.current_step >= c.profile_start_at_step + c.profile_steps - 1:
            if self.observations:
                self.save()

    def save(self) -> None:
        self._saved = True
        rows = [tuple(o) for o in self.observations]
        if dist.is_initialized() and self.topology.world_size > 1:
            gathered: Optional[list] = [None] * self.topology.world_size if self.topology.config.global_rank == 0 else None
            dist.gather_object(rows, gathered, dst=0)
        else:
            gathered = [rows]
        if self.topology.config.global_rank in (0, None) and self.config.profiler_output is not None:
            out = Path(self.config.profiler_output)
            out.parent.mkdir(parents=True, exist_ok=True)
            # top-level sizes and one dict per observation as in src/scaling/core/profiler/profiler.py:94-101; the
            # whole topology config in addition
            tc = self.topology.config
            fields = list(ProfilerObservation._fields)
            rows = [r for part in (gathered or []) for r in (part or [])]
            payload = {
                "pipe_parallel_size": tc.pipe_parallel_size, "data_parallel_size": tc.data_parallel_size,
                "model_parallel_size": tc.model_parallel_size,
                "gradient_accumulation_steps": tc.gradient_accumulation_steps,
                "topology": tc.as_dict(),
                "fields": fields,
                "observations": [dict(zip(fields, r)) if isinstance(r, (list, tuple)) else r for r in rows],
            }
            out.write_text(json.dumps(payload))

    def start_timer(self, timer_name: str, micro_batch_id: Optional[int] = None, buffer_id: Optional[int] = None) -> None:
        if not self.active:
            return
        timer = CudaEventTimer()
        self._open[(timer_name, micro_batch_id, buffer_id)] = timer
        timer.start()

    def stop_timer(self, timer_name: str, micro_batch_id: Optional[int] = None, buffer_id: Optional[int] = None) -> None:
        timer = self._open.pop((timer_name, micro_batch_id, buffer_id), None)
        if timer is None:
            return
        timer.stop()
        self._pending.append((timer_name, self.current_step, micro_batch_id, buffer_id, timer))

    @contextlib.contextmanager
    def time(self, timer_name: str, micro_batch_id: Optional[int] = None, buffer_id: Optional[int] = None) -> Iterator[None]:
        self.start_timer(timer_name, micro_batch_id, buffer_id)
        try:
            yield
        finally:
            self.stop_timer(timer_name, micro_batch_id, buffer_id)
