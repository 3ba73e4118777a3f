"""Linear layer with operands rounded to FP8 per matmul.

Each of the three products (forward ``x w^T``, ``grad_y w`` and ``grad_y^T x``) rounds its two
operands to the configured fp8 formats with saturation and without scaling factors, exactly what
the reference's ``fp8_linear`` feeds to ``torch._scaled_mm`` (src/scaling/core/fp8/fp8_linear.py:10-110);
a product whose dtype pair is ``None`` runs unquantised.  On a GPU the rounded operands go to the fp8
tensor-core GEMM (``tcgen05.mma kind::f8f6f4``, fp32 accumulation in TMEM), which is the scaled-mm result with
unit scales; on CPU ranks, and for shapes whose reduction length is not a multiple of 16, they are widened and
multiplied in the compute dtype, which gives the same values.
"""

from __future__ import annotations

from typing import Optional

import torch

from ...ops import functional as K


def saturating_cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    lim = torch.finfo(dtype).max
    return x.clamp(min=-lim, max=lim).to(dtype)


def _round(x: torch.Tensor, dtype: Optional[torch.dtype]) -> torch.Tensor:
    if dtype is None or x.dtype == dtype:
        return x if x.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2) else x
    return saturating_cast(x, dtype)


def _mm(a: torch.Tensor, b_t: torch.Tensor, compute: torch.dtype) -> torch.Tensor:
    """``a @ b_t.T``: on the fp8 tensor cores when both operands are fp8, else widened to ``compute``."""
    if a.is_cuda and compute == torch.bfloat16:
        a, b_t = a.contiguous(), b_t.contiguous()
        if K.gemm_fp8_supported(a, b_t):
            return K.gemm_fp8(a, b_t, out_dtype=compute)
    return K.gemm(a.to(compute).contiguous(), b_t.to(compute).contiguous()) if a.is_cuda and compute != torch.float32 \
        else a.to(compute) @ b_t.to(compute).t()


class _FP8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, dt_fwd, dt_gi, dt_gw):  # type: ignore[override]
        compute = x.dtype if x.dtype in (torch.bfloat16, torch.float16) else torch.float32
        x2 = x.reshape(-1, x.shape[-1])
        xq = _round(x2, dt_fwd[0]) if dt_fwd else x2
        wq = _round(w, dt_fwd[1]) if dt_fwd else w
        y = _mm(xq, wq, compute)
        if bias is not None:
            y = y + bias.to(y.dtype)
        ctx.save_for_backward(x2, w)
        ctx.cfg = (dt_gi, dt_gw, compute, bias is not None, x.shape)
        return y.view(*x.shape[:-1], w.shape[0]).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x2, w = ctx.saved_tensors
        dt_gi, dt_gw, compute, has_bias, x_shape = ctx.cfg
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            g = _round(dy2, dt_gi[0]) if dt_gi else dy2
            wq = _round(w, dt_gi[1]) if dt_gi else w
            dx = _mm(g, wq.t().contiguous(), compute).view(x_shape).to(dy.dtype)
        if ctx.needs_input_grad[1]:
            xq = _round(x2, dt_gw[0]) if dt_gw else x2
            g = _round(dy2, dt_gw[1]) if dt_gw else dy2
            dw = _mm(g.t().contiguous(), xq.t().contiguous(), compute)
            dw = dw.to(w.dtype if w.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2) else dy.dtype)
        if has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db, None, None, None


E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2


def fp8_linear(input: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,  # noqa: A002
               dtypes_forward: Optional[tuple[torch.dtype, torch.dtype]] = (E4M3, E4M3),
               dtypes_grad_input: Optional[tuple[torch.dtype, torch.dtype]] = (E5M2, E4M3),
               dtypes_grad_weight: Optional[tuple[torch.dtype, torch.dtype]] = (E4M3, E5M2)) -> torch.Tensor:
    """Signature and defaults of src/scaling/core/fp8/fp8_linear.py:76-83: e4m3 operands forward, e5m2 for the
    incoming gradient in both backward products; ``None`` for a pair leaves that product unquantised."""
    return _FP8Linear.apply(input, weight, bias, dtypes_forward, dtypes_grad_input, dtypes_grad_weight)


to_fp8_saturated = saturating_cast  # the name in src/scaling/core/fp8/fp8_linear.py:10
