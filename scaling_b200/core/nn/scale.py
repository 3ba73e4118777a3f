"""Scalar multiplications that act in only one direction of autograd.

``scale_fwd(x, s)`` multiplies the activation, ``scale_bwd(x, s)`` multiplies the gradient
(unit-scaling primitives used by u-muP; reference: src/scaling/core/nn/scale.py:13-74).
"""

from __future__ import annotations

import torch


class _DirectionalScale(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, fwd, bwd) -> torch.Tensor:  # type: ignore[override]
        ctx.bwd = bwd
        if torch.is_tensor(fwd):
            return x * fwd.to(x.dtype)
        return x if fwd == 1.0 else x * fwd

    @staticmethod
    def backward(ctx, g: torch.Tensor):  # type: ignore[override]
        if torch.is_tensor(ctx.bwd):
            return g * ctx.bwd.to(g.dtype), None, None
        return (g if ctx.bwd == 1.0 else g * ctx.bwd), None, None


def _factor(scale):
    """A Python number, or a 0-dim tensor that stays on its device (no host synchronisation, no gradient)."""
    return scale.detach() if torch.is_tensor(scale) else float(scale)


def scale_fwd(input: torch.Tensor, scale) -> torch.Tensor:  # noqa: A002
    return _DirectionalScale.apply(input, _factor(scale), 1.0)


def scale_bwd(input: torch.Tensor, scale) -> torch.Tensor:  # noqa: A002
    return _DirectionalScale.apply(input, 1.0, _factor(scale))
