"""Scalar multiplications that act in only one direction of autograd.

``scale_fwd(x, s)`` multiplies the activation, ``scale_bwd(x, s)`` multiplies the gradient
(unit-scaling primitives used by u-muP; reference: src/scaling/core/nn/scale.py:13-74).
"""

from __future__ import annotations

import torch


class _DirectionalScale(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, fwd: float, bwd: float) -> torch.Tensor:  # type: ignore[override]
        ctx.bwd = bwd
        return x if fwd == 1.0 else x * fwd

    @staticmethod
    def backward(ctx, g: torch.Tensor):  # type: ignore[override]
        return (g if ctx.bwd == 1.0 else g * ctx.bwd), None, None


def scale_fwd(x: torch.Tensor, scale: float) -> torch.Tensor:
    return _DirectionalScale.apply(x, float(scale), 1.0)


def scale_bwd(x: torch.Tensor, scale: float) -> torch.Tensor:
    return _DirectionalScale.apply(x, 1.0, float(scale))
