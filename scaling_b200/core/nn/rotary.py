"""Rotary position embeddings.

Two conventions, as in the reference (src/scaling/core/nn/rotary.py:142-255):
``RotaryEmbedding`` pairs element ``i`` with ``i + d/2`` ("rotate half", GPT-NeoX layout) and may
rotate only the first ``dimensions`` of each head; ``RotaryEmbeddingComplex`` pairs ``2i`` with
``2i + 1`` (Llama layout).  Both accept ``[seq, batch, heads, head_dim]`` tensors and optional
``[seq, batch]`` position ids.  Angles are evaluated in fp32 inside one fused kernel that rotates in
place on a contiguous copy; no cos/sin table is materialised (the reference caches the rotate-half
table in the model dtype, so bf16 results differ in the last bit).
"""

from __future__ import annotations

from typing import Optional

import torch
from pydantic import Field

from ...ops import functional as K
from ..config import BaseConfig


class RotaryConfig(BaseConfig):
    dimensions: int = Field(0, description="number of leading head dimensions that are rotated")
    base: int = Field(10000, description="base of the geometric frequency progression")
    max_seq_length: int = Field(2048, description="longest sequence (kept for config compatibility)")


def apply_rotary_tokens(x: torch.Tensor, positions: torch.Tensor, dimensions: int, base: float,
                        interleaved: bool) -> torch.Tensor:
    """``x``: ``[tokens, heads, head_dim]``; ``positions``: ``[tokens]``."""
    return K.rope(x, positions, dimensions, float(base), interleaved)


def _positions_for(x_sbhd: torch.Tensor, position_ids: Optional[torch.Tensor]) -> torch.Tensor:
    s, b = x_sbhd.shape[0], x_sbhd.shape[1]
    if position_ids is None:
        return torch.arange(s, device=x_sbhd.device, dtype=torch.int32).repeat_interleave(b)
    # [s, b], the token order of the [s, b, ...] tensor (src/scaling/core/nn/attention/attention.py:838-844 turns the
    # batch's [b, s] ids around before it calls the module)
    assert position_ids.shape == (s, b), f"position ids {tuple(position_ids.shape)} for activations [{s}, {b}, ...]"
    return position_ids.reshape(-1)


class _RotaryBase(torch.nn.Module):
    interleaved = False

    def __init__(self, config: RotaryConfig, device: Optional[torch.device] = None,
                 dtype: torch.dtype = torch.float32) -> None:
        super().__init__()
        assert config.dimensions > 1, "RotaryEmbedding cannot use `dim` == 1, this results in weird reshape errors"
        self.dimensions = config.dimensions
        self.base = float(config.base)
        self.max_seq_length = config.max_seq_length

    def _one(self, x: torch.Tensor, position_ids: Optional[torch.Tensor]) -> torch.Tensor:
        assert x.shape[-1] >= self.dimensions, f"head dim {x.shape[-1]} < rotary dims {self.dimensions}"
        s, b, h, d = x.shape
        out = apply_rotary_tokens(x.reshape(s * b, h, d), _positions_for(x, position_ids), self.dimensions,
                                  self.base, self.interleaved)
        return out.view(s, b, h, d)

    def forward(self, query: torch.Tensor, key: torch.Tensor, query_position_ids: Optional[torch.Tensor] = None,
                key_position_ids: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
        return self._one(query, query_position_ids), self._one(key, key_position_ids)


class RotaryEmbedding(_RotaryBase):
    interleaved = False


class RotaryEmbeddingComplex(_RotaryBase):
    interleaved = True

    def __init__(self, config: RotaryConfig, device: Optional[torch.device] = None) -> None:
        super().__init__(config, device)
