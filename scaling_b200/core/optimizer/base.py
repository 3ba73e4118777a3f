"""Optimizer interface of the engine (src/scaling/core/optimizer/base.py:10-88)."""

from __future__ import annotations

from abc import ABC, abstractmethod
from pathlib import Path
from typing import Any, Dict, NamedTuple, Optional

import torch

from ..config import BaseConfig


class OptimizerStepOutput(NamedTuple):
    global_grad_norm: Optional[float]
    global_grad_norm_clipped: Optional[float]
    learning_rates: Optional[Dict[str, float]]
    overflow: Optional[bool]
    no_overflow_steps: Optional[int]
    current_loss_scale: Optional[float]
    debug_dict: Optional[Dict[str, float]]


class BaseOptimizer(ABC):
    def __init__(self, config: BaseConfig) -> None:
        self.config = config

    def __repr__(self) -> str:
        return type(self).__name__

    @abstractmethod
    def step(self) -> OptimizerStepOutput:
        """Update the parameters from the accumulated gradients and clear the gradients."""

    @abstractmethod
    def backward(self, loss: torch.Tensor) -> None:
        """Backward pass on a micro-batch loss, including gradient-accumulation and loss scaling."""

    @abstractmethod
    def state_dict(self) -> dict[str, Any]:
        ...

    @abstractmethod
    def save_checkpoint(self, dir: Path) -> None:
        ...

    @abstractmethod
    def load_checkpoint(self, dir: Path) -> None:
        ...

    @abstractmethod
    def refresh_optimizer_after_model_change(self) -> None:
        """Re-derive the full-precision master copies after the model weights were changed from outside."""

    def log_state(self) -> None:
        pass
