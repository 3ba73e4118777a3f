"""Instruction set of the pipeline engine (src/scaling/core/nn/pipeline_schedule/instructions.py:5-61)."""

from __future__ import annotations

from typing import NamedTuple, Optional


class InstructionBase(NamedTuple):
    buffer_id: Optional[int] = None
    micro_batch_id: Optional[int] = None
    is_first_pass: Optional[bool] = None

    @property
    def name(self) -> str:
        return type(self).__name__.removeprefix("Instruction")


def _instruction(name: str) -> type:
    return type(name, (InstructionBase,), {"__slots__": ()})


InstructionOptimizerStep = _instruction("InstructionOptimizerStep")
InstructionReduceTiedGrads = _instruction("InstructionReduceTiedGrads")
InstructionStoreMicroBatch = _instruction("InstructionStoreMicroBatch")
InstructionLoadMicroBatch = _instruction("InstructionLoadMicroBatch")
InstructionForwardPass = _instruction("InstructionForwardPass")
InstructionLoss = _instruction("InstructionLoss")
InstructionBackwardPass = _instruction("InstructionBackwardPass")
InstructionSendActivation = _instruction("InstructionSendActivation")
InstructionRecvActivation = _instruction("InstructionRecvActivation")
InstructionSendGrad = _instruction("InstructionSendGrad")
InstructionRecvGrad = _instruction("InstructionRecvGrad")

# a communication instruction completes together with this instruction on the neighbouring stage
# (offset -1 = previous stage, +1 = next stage)
PEER_OF = {
    "SendActivation": ("RecvActivation", +1),
    "RecvActivation": ("SendActivation", -1),
    "SendGrad": ("RecvGrad", -1),
    "RecvGrad": ("SendGrad", +1),
}
