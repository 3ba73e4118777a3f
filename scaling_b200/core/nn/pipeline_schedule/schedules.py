"""Pipeline schedules: 1F1B for training, fill-drain for inference.

Training (src/scaling/core/nn/pipeline_schedule/train.py:32-174): ``2 * (grad_acc + pp - 1)`` clock
ticks; even stages run forwards on even ticks and backwards on odd ticks, odd stages the other way
round, which interleaves one forward with one backward in the steady state.  A tick emits, in order:
communication (forward tick: receive this micro batch's activation, then send the previous one's
gradient; backward tick: send the previous activation, then receive this gradient), the data load on
the first/last stage, and the compute instruction(s).  The last tick appends the tied-gradient
reduction and the optimizer step.  Micro batch ``m`` uses buffer ``m % max(2, min(pp - stage + 1, ga))``.

Inference (src/scaling/core/nn/pipeline_schedule/inference.py:16-75): ``grad_acc + pp - 1`` ticks,
micro batch ``tick - stage``, two buffers alternating by tick parity; even stages send before they
receive, odd stages receive before they send, so neighbouring stages always rendezvous.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Optional

from ....parallel.topology import Topology
from .instructions import (
    InstructionBackwardPass,
    InstructionBase,
    InstructionForwardPass,
    InstructionLoadMicroBatch,
    InstructionLoss,
    InstructionOptimizerStep,
    InstructionRecvActivation,
    InstructionRecvGrad,
    InstructionReduceTiedGrads,
    InstructionSendActivation,
    InstructionSendGrad,
)


class PipelineScheduleBase(ABC):
    def __init__(self, topology: Topology):
        self.topology = topology
        self.stage = topology.pipe_parallel_rank
        self.stages = topology.config.pipe_parallel_size
        self.micro_batches = topology.config.gradient_accumulation_steps

    @abstractmethod
    def instructions(self) -> list[InstructionBase]:
        ...

    @abstractmethod
    def required_buffer_count(self) -> int:
        ...

    def _valid_micro_batch(self, micro_batch_id: int) -> bool:
        return 0 <= micro_batch_id < self.micro_batches

    def _is_valid_pipe_parallel_rank(self, pipe_parallel_rank: Optional[int]) -> bool:
        return pipe_parallel_rank is not None and 0 <= pipe_parallel_rank < self.stages

    @property
    def has_previous(self) -> bool:
        return self.stage > 0

    @property
    def has_next(self) -> bool:
        return self.stage < self.stages - 1

    @property
    def loads_data(self) -> bool:
        return self.stage == 0 or self.stage == self.stages - 1

    # simulation / drawing helpers live in simulator.py; thin forwards keep the reference's entry points
    @classmethod
    def illustrate(cls, gradient_accumulation_steps: int, pipe_parallel_size: int) -> dict:
        from .simulator import illustrate

        return illustrate(cls, gradient_accumulation_steps, pipe_parallel_size)

    @classmethod
    def visualize(cls, gradient_accumulation_steps: int, pipe_parallel_size: int):
        from .simulator import visualize_lockstep

        return visualize_lockstep(cls, gradient_accumulation_steps, pipe_parallel_size)

    @classmethod
    def visualize_profile(cls, profile_file, milliseconds_per_pixel: float = 10, pipe_pixels: int = 200):
        from .simulator import SimulationEngine

        engine = SimulationEngine.from_profile(cls, profile_file)
        engine.simulate()
        # (summary of the simulated run, timeline image), as src/scaling/core/nn/pipeline_schedule/base.py:222-239
        return engine.summarize(), engine.visualize(milliseconds_per_pixel=milliseconds_per_pixel,
                                                   pipe_pixels=pipe_pixels)


class PipelineScheduleTrain(PipelineScheduleBase):
    def required_buffer_count(self) -> int:
        return max(2, min(self.stages - self.stage + 1, self.micro_batches))

    def _buffer_idx(self, micro_batch_id: int) -> int:
        return micro_batch_id % self.required_buffer_count()

    def _tick(self, tick: int) -> tuple[int, bool]:
        """(micro batch, is_forward) this stage works on at clock ``tick``; the id may be out of range."""
        r, pp = self.stage, self.stages
        forward = (tick % 2) == (r % 2)
        half = tick // 2  # also (tick - 1) // 2 for odd ticks
        if forward:
            return half - r // 2, True
        if tick % 2 == 0:  # odd stage, even tick
            return half - pp + (r + 1) // 2, False
        return half - pp + 1 + r // 2, False  # even stage, odd tick

    def instructions(self) -> list[InstructionBase]:
        out: list[InstructionBase] = []
        ticks = 2 * (self.micro_batches + self.stages - 1)
        prev_mb = -1
        for tick in range(ticks):
            mb, forward = self._tick(tick)
            cur_ok, prev_ok = self._valid_micro_batch(mb), self._valid_micro_batch(prev_mb)
            cur_buf = self._buffer_idx(mb) if cur_ok else None
            prev_buf = self._buffer_idx(prev_mb) if prev_ok else None
            if forward:
                if cur_ok and self.has_previous:
                    out.append(InstructionRecvActivation(buffer_id=cur_buf, micro_batch_id=mb))
                if prev_ok and self.has_previous:
                    out.append(InstructionSendGrad(buffer_id=prev_buf, micro_batch_id=prev_mb))
            else:
                if prev_ok and self.has_next:
                    out.append(InstructionSendActivation(buffer_id=prev_buf, micro_batch_id=prev_mb))
                if cur_ok and self.has_next:
                    out.append(InstructionRecvGrad(buffer_id=cur_buf, micro_batch_id=mb))
            if cur_ok and forward and self.loads_data:
                out.append(InstructionLoadMicroBatch(buffer_id=cur_buf, micro_batch_id=mb))
            if cur_ok:
                if forward:
                    out.append(InstructionForwardPass(buffer_id=cur_buf, micro_batch_id=mb))
                    if not self.has_next:
                        out.append(InstructionLoss(buffer_id=cur_buf, micro_batch_id=mb, is_first_pass=True))
                else:
                    out.append(InstructionBackwardPass(buffer_id=cur_buf, micro_batch_id=mb))
            prev_mb = mb
        out.append(InstructionReduceTiedGrads())
        out.append(InstructionOptimizerStep())
        return out


class PipelineScheduleInference(PipelineScheduleBase):
    def required_buffer_count(self) -> int:
        return 2

    def instructions(self) -> list[InstructionBase]:
        out: list[InstructionBase] = []
        even = self.stage % 2 == 0
        for tick in range(self.micro_batches + self.stages - 1):
            mb = tick - self.stage
            recv_buf = tick % 2 if even else (tick + 1) % 2
            send_buf = 1 - recv_buf
            cur_ok = self._valid_micro_batch(mb)
            prev_ok = self._valid_micro_batch(mb - 1)
            if cur_ok and self.loads_data:
                out.append(InstructionLoadMicroBatch(buffer_id=recv_buf, micro_batch_id=mb))
            send = InstructionSendActivation(buffer_id=send_buf, micro_batch_id=mb) if (self.has_next and prev_ok) else None
            recv = InstructionRecvActivation(buffer_id=recv_buf, micro_batch_id=mb) if (self.has_previous and cur_ok) else None
            for ins in ((send, recv) if even else (recv, send)):
                if ins is not None:
                    out.append(ins)
            if cur_ok:
                out.append(InstructionForwardPass(buffer_id=recv_buf, micro_batch_id=mb))
                if not self.has_next:
                    out.append(InstructionLoss(buffer_id=recv_buf, micro_batch_id=mb))
        return out
