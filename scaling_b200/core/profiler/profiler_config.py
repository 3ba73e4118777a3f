"""Profiler settings (fields of src/scaling/core/profiler/profiler_config.py:9-24)."""

from pathlib import Path
from typing import Optional

from pydantic import Field

from ..config import BaseConfig


class ProfilerConfig(BaseConfig):
    profile_steps: int = Field(0, description="number of steps to time; 0 disables profiling")
    profile_start_at_step: int = Field(10, description="first step that is timed (lets warm-up pass)")
    profiler_output: Optional[Path] = Field(None, description="json file that receives the gathered observations")
