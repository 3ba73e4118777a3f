"""Dynamic loss scaling for fp16 training.

State machine of src/scaling/core/optimizer/loss_scaler.py:83-113: on overflow the scale is divided
by ``factor`` (not below ``min_scale``) once the hysteresis budget is used up, and the step is
skipped; after ``window`` consecutive clean steps the scale is multiplied by ``factor``.  Overflow
detection itself happens on the device: the gradient-norm kernel raises a sticky inf/nan flag that
travels with the norm in one all-reduce, so there is no per-parameter host synchronisation.
"""

from __future__ import annotations

from typing import NamedTuple, Optional, TypedDict

import torch
from pydantic import Field

from ..config import BaseConfig


class LossScalerConfig(BaseConfig):
    """Dynamic loss scaling: start high, halve on overflow (and skip the step), double after a
    window of clean steps."""

    enable: bool = Field(False, description="scale the loss before backward")
    initial_scale: float = Field(2.0 ** 32, description="initial loss scale")
    window: int = Field(1000, description="clean steps after which the scale grows")
    hysteresis: float = Field(2, description="overflows tolerated before the scale shrinks")
    consecutive_hysteresis: bool = Field(False, description="refill the hysteresis budget after every clean step")
    min_scale: float = Field(1.0, description="lower bound of the scale")
    factor: float = Field(2.0, description="growth / shrink factor")


class LossScalerState(TypedDict):
    current_scale: float
    current_hysteresis: float
    no_overflow_steps: int


class LossScalerOutput(NamedTuple):
    overflow: Optional[bool]
    no_overflow_steps: Optional[int]
    current_loss_scale: Optional[float]


class LossScaler:
    def __init__(self, config: LossScalerConfig, parameter_groups: Optional[list] = None,
                 parameters: Optional[list[torch.Tensor]] = None):
        # The gradients are not needed here: overflow is detected on the device inside the optimizer step and handed
        # to ``step``; the arguments keep the constructor of src/scaling/core/optimizer/loss_scaler.py callable as is.
        self.config = config
        self._current_scale = config.initial_scale
        self._current_hysteresis = config.hysteresis
        self._no_overflow_steps = 0

    @property
    def current_scale(self) -> float:
        return self._current_scale if self.config.enable else 1.0

    def state_dict(self) -> LossScalerState:
        return {
            "current_scale": self._current_scale,
            "current_hysteresis": self._current_hysteresis,
            "no_overflow_steps": self._no_overflow_steps,
        }

    def load_state_dict(self, state_dict: LossScalerState) -> None:
        self._current_scale = state_dict["current_scale"]
        self._current_hysteresis = state_dict["current_hysteresis"]
        self._no_overflow_steps = state_dict["no_overflow_steps"]

    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self._current_scale if self.config.enable else loss

    def step(self, overflow: bool) -> LossScalerOutput:
        """Advance the state machine with this step's overflow verdict (already agreed on by all ranks)."""
        c = self.config
        if not c.enable:
            return LossScalerOutput(None, None, None)
        if overflow:
            if c.hysteresis == 1 or self._current_hysteresis == 1:
                self._current_scale = max(self._current_scale / c.factor, c.min_scale)
            else:
                self._current_hysteresis -= 1
            self._no_overflow_steps = 0
        else:
            if c.consecutive_hysteresis:
                self._current_hysteresis = c.hysteresis
            if self._no_overflow_steps > 0 and self._no_overflow_steps % c.window == 0:
                if not c.consecutive_hysteresis:
                    self._current_hysteresis = c.hysteresis
                self._current_scale *= c.factor
            self._no_overflow_steps += 1
        return LossScalerOutput(overflow, self._no_overflow_steps, self._current_scale)
