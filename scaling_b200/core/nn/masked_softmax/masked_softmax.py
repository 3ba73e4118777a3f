"""Scaled, masked softmax over attention scores.

``softmax(masked_fill(x * scale, mask, -10000))`` with optional fp32 evaluation - the torch path
of the reference (src/scaling/core/nn/masked_softmax/masked_softmax.py:8-52) - as one fused kernel
on GPUs (fp32 math always).  ``kernel = flash_attention`` selects the fused attention kernel in
``ParallelSelfAttention``, where the softmax never materialises.
"""

from __future__ import annotations

from enum import Enum
from typing import Optional

import torch
from pydantic import Field

from ....ops import functional as K
from ...config import BaseConfig


class MaskedSoftmaxKernel(Enum):
    TORCH = "torch"
    FLASH_ATTENTION = "flash_attention"


class MaskedSoftmaxConfig(BaseConfig):
    kernel: MaskedSoftmaxKernel = Field(MaskedSoftmaxKernel.TORCH, description="attention implementation")
    softmax_in_fp32: bool = Field(False, description="evaluate the softmax in fp32 (always true on GPUs)")
    scale: float = Field(1.0, description="factor applied to the scores before the softmax")
    deterministic_flash_attn_bwd: bool = Field(
        False, description="kept for config compatibility; the fused attention backward is always deterministic"
    )


class MaskedSoftmax(torch.nn.Module):
    def __init__(self, config: MaskedSoftmaxConfig):
        super().__init__()
        self.config = config

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor]) -> torch.Tensor:
        return K.masked_softmax(x, mask, self.config.scale, self.config.softmax_in_fp32)
