"""Learning-rate schedule: delay -> linear warm-up -> {constant, linear, cosine} decay -> floor.

For the 1-based step ``t``: 0 while ``t <= delay``; ``lr * (t - delay) / warmup`` during warm-up; then
``min + coeff * (lr - min)`` with ``ratio = (t - warmup - delay) / (decay_iters - warmup - delay)`` and
``coeff = 1 - ratio`` (linear) or ``(cos(pi * ratio) + 1) / 2`` (cosine); ``min`` once ``t`` exceeds
``decay_iters`` (src/scaling/core/optimizer/learning_rate_scheduler/learning_rate_scheduler.py:9-66).
"""

from __future__ import annotations

import math
from enum import Enum

from pydantic import Field

from ...config import BaseConfig


class LearningRateDecayStyle(Enum):
    CONSTANT = "constant"
    LINEAR = "linear"
    COSINE = "cosine"


class LearningRateSchedulerConfig(BaseConfig):
    learning_rate: float = Field(0.0, description="base (= maximum) learning rate")
    learning_rate_minimum: float = Field(0.0, description="floor of the schedule")
    learning_rate_decay_style: LearningRateDecayStyle = Field(
        LearningRateDecayStyle.COSINE, description="shape of the decay after warm-up"
    )
    learning_rate_decay_iters: int = Field(0, description="iterations over which the schedule runs (incl. warm-up)")
    learning_rate_warmup_steps: int = Field(0, description="linear warm-up steps")
    learning_rate_warmup_delay_steps: int = Field(0, description="steps at zero learning rate before warm-up")


class LearningRateScheduler:
    def __init__(self, config: LearningRateSchedulerConfig):
        self.config = config

    def get_lr(self, step_index: int) -> float:
        c = self.config
        delay, warmup = c.learning_rate_warmup_delay_steps, c.learning_rate_warmup_steps
        if step_index <= delay:
            return 0.0
        if warmup > 0 and step_index <= warmup + delay:
            return c.learning_rate * (step_index - delay) / warmup
        if c.learning_rate_decay_style == LearningRateDecayStyle.CONSTANT:
            return c.learning_rate
        if step_index > c.learning_rate_decay_iters:
            return c.learning_rate_minimum
        span = c.learning_rate_decay_iters - warmup - delay
        ratio = (step_index - warmup - delay) / span if span > 0 else 1.0
        assert 0.0 <= ratio <= 1.0
        if c.learning_rate_decay_style == LearningRateDecayStyle.LINEAR:
            coeff = 1.0 - ratio
        elif c.learning_rate_decay_style == LearningRateDecayStyle.COSINE:
            coeff = 0.5 * (math.cos(math.pi * ratio) + 1.0)
        else:
            raise NotImplementedError(f"{c.learning_rate_decay_style} decay style is not supported.")
        return c.learning_rate_minimum + coeff * (c.learning_rate - c.learning_rate_minimum)
