"""Residual split / add with optional u-muP scaling of the branch and the skip path
(reference: src/scaling/core/nn/residual.py:9-65)."""

from __future__ import annotations

from typing import Any, Optional

import torch

from .scale import scale_bwd, scale_fwd
from .umup import UMuParametrization


class _ResidualOp(torch.nn.Module):
    def __init__(self, umup_residual_mults: Optional[list[float]] = None,
                 umup_residual_layer_index: Optional[int] = None, umup_pre_norm: Optional[bool] = None) -> None:
        super().__init__()
        self.umup_residual_mults = umup_residual_mults
        self.umup_residual_layer_index = umup_residual_layer_index
        self.umup_pre_norm = umup_pre_norm
        self._use_umup = False
        self.residual_scale = 1.0
        self.skip_scale = 1.0

    def umup_setup(self, depth: int, **kwargs: Any) -> None:
        assert self.umup_residual_mults is not None and self.umup_residual_layer_index is not None
        assert self.umup_pre_norm is not None
        self.residual_scale, self.skip_scale = UMuParametrization.get_umup_residual_scales(
            self.umup_residual_mults, self.umup_residual_layer_index, self.umup_pre_norm, depth
        )
        self._use_umup = True


class NormedResidualSplit(_ResidualOp):
    def forward(self, hidden_state: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        if not self._use_umup:
            return hidden_state, hidden_state
        return scale_bwd(hidden_state, self.residual_scale), scale_bwd(hidden_state, self.skip_scale)


class NormedResidualAdd(_ResidualOp):
    def forward(self, hidden_state_residual: torch.Tensor, hidden_state_skip: torch.Tensor) -> torch.Tensor:
        if self._use_umup:
            hidden_state_residual = scale_fwd(hidden_state_residual, self.residual_scale)
            hidden_state_skip = scale_fwd(hidden_state_skip, self.skip_scale)
        return hidden_state_residual + hidden_state_skip
