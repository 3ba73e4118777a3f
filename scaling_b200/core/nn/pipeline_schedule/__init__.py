from .instructions import *  # noqa: F401,F403
from .instructions import InstructionBase
from .schedules import PipelineScheduleBase, PipelineScheduleInference, PipelineScheduleTrain
from .simulator import SimulationEngine, SimulationInstruction, illustrate

__all__ = ["InstructionBase", "PipelineScheduleBase", "PipelineScheduleInference", "PipelineScheduleTrain",
           "SimulationEngine", "SimulationInstruction", "illustrate"]
