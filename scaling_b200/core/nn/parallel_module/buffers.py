"""Micro-batch slots of one pipeline stage (src/scaling/core/nn/parallel_module/buffers.py:8-46)."""

from __future__ import annotations

from enum import Enum
from typing import Any, Optional

import torch


class BufferType(Enum):
    PIPELINE_STAGE_INPUT = "pipeline_stage_input"
    PIPELINE_STAGE_OUTPUT = "pipeline_stage_output"
    TARGET = "target"
    LOSS = "loss"
    METRICS = "metrics"
    GRAD = "grad"


class Buffers:
    def __init__(self) -> None:
        self._slots: dict[BufferType, dict[int, Any]] = {t: {} for t in BufferType}
        self.losses: list[torch.Tensor] = []
        self.metrics: list[dict[str, torch.Tensor]] = []

    def reset(self) -> None:
        for d in self._slots.values():
            d.clear()
        self.losses = []
        self.metrics = []

    def write(self, buffer_type: BufferType, buffer_id: int, data: Any) -> None:
        self._slots[buffer_type][buffer_id] = data

    def get(self, buffer_type: BufferType, buffer_id: int) -> Any:
        return self._slots[buffer_type][buffer_id]

    def has(self, buffer_type: BufferType, buffer_id: int) -> bool:
        return buffer_id in self._slots[buffer_type]

    def take(self, buffer_type: BufferType, buffer_id: int) -> Any:
        """Return the slot's content and free the slot."""
        return self._slots[buffer_type].pop(buffer_id)

    def dump(self, buffer_type: BufferType, buffer_id: int) -> None:
        self._slots[buffer_type].pop(buffer_id, None)

    def add_loss(self, loss: torch.Tensor, metrics: Optional[dict[str, torch.Tensor]] = None) -> None:
        self.losses.append(loss.detach())
        if metrics is not None:
            self.metrics.append({k: (v.detach() if isinstance(v, torch.Tensor) else v) for k, v in metrics.items()})
