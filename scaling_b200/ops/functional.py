"""Functional front end of the sm_100a kernels (autograd aware).

Every op has two bodies: the CUDA kernel from ``libsb200.so`` (used whenever the tensors live on a
GPU) and a plain torch expression (used by CPU/gloo ranks and as the oracle in tests).  The kernel
path never silently degrades on a GPU: unsupported dtypes raise, and only shapes that violate a
kernel's vector-width contract take the torch expression.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import check, dt, lib, ptr, sm_count, stream

_KERNEL_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def on_gpu(*ts: Optional[torch.Tensor]) -> bool:
    return any(t is not None and t.is_cuda for t in ts)


# --------------------------------------------------------------------------- status word
_STATUS: dict[int, torch.Tensor] = {}


def status_word() -> torch.Tensor:
    """Per-device int32 that kernels with bounded waits set when a wait expires."""
    d = torch.cuda.current_device()
    if d not in _STATUS:
        _STATUS[d] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{d}")
    return _STATUS[d]


def check_status() -> None:
    """Synchronising read of the status word; raises CommTimeout if a device-side wait gave up."""
    if not torch.cuda.is_available():
        return
    d = torch.cuda.current_device()
    if d in _STATUS:
        v = int(_STATUS[d].item())
        if v != 0:
            _STATUS[d].zero_()
            if d in _GEMM_WS:
                _GEMM_WS[d][:4096].zero_()  # an aborted split-K launch may have left tile counters behind
            check(v, "device status word")


# --------------------------------------------------------------------------- GEMM
def _gemm_ok(a: torch.Tensor, b: torch.Tensor) -> bool:
    return (
        a.is_cuda
        and a.dtype in (torch.bfloat16, torch.float16)
        and b.dtype == a.dtype
        and a.dim() == 2
        and b.dim() == 2
        and a.stride(1) == 1
        and b.stride(1) == 1
        and a.stride(0) % 8 == 0
        and b.stride(0) % 8 == 0
        and a.data_ptr() % 16 == 0
        and b.data_ptr() % 16 == 0
    )


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_mn: bool = False,
    b_mn: bool = False,
    bias: Optional[torch.Tensor] = None,
    act: str = "none",
    out: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    out_dtype: Optional[torch.dtype] = None,
    pre_act_out: Optional[torch.Tensor] = None,
    bn: int = 0,
    split: int = 0,
) -> torch.Tensor:
    """``C = op(a) @ op(b)^T``-style GEMM on tcgen05.

    ``a`` is ``[M, K]`` (``a_mn=False``) or ``[K, M]`` (``a_mn=True``); ``b`` is ``[N, K]``
    (``b_mn=False``) or ``[K, N]`` (``b_mn=True``).  Result ``[M, N]``.
    """
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    odt = out_dtype or (out.dtype if out is not None else a.dtype)
    kernel = _gemm_ok(a, b) and not (a_mn and not b_mn) and K > 0 and M > 0 and N > 0
    if kernel and out is not None and (out.stride(1) != 1 or out.dim() != 2):
        kernel = False
    if kernel and odt not in (torch.float32, a.dtype):
        kernel = False
    if kernel and bias is not None and (bias.dtype != a.dtype or not bias.is_contiguous()):
        bias = bias.to(a.dtype).contiguous()
    if not kernel:
        if a.is_cuda and a.dtype in (torch.bfloat16, torch.float16) and not _gemm_shape_exempt(a, b):
            raise _lib.KernelError(
                f"gemm: operands not accepted by the tcgen05 kernel (shapes {tuple(a.shape)} {tuple(b.shape)}, "
                f"strides {a.stride()} {b.stride()})"
            )
        am = a.t() if a_mn else a
        bm = b if b_mn else b.t()
        c = (am.float() @ bm.float()) if a.dtype != torch.float32 else am @ bm
        if bias is not None:
            c = c + bias.float()
        if pre_act_out is not None:
            pre_act_out.copy_(c)
        if act == "gelu":
            c = F.gelu(c)
        if out is not None:
            if accumulate:
                out.add_(c.to(out.dtype))
            else:
                out.copy_(c)
            return out
        return c.to(odt)
    if out is None:
        out = torch.empty((M, N), dtype=odt, device=a.device)
        assert not accumulate
    ws = _gemm_workspace(a.device)
    rc = lib().sb200_gemm_ws(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), ptr(pre_act_out), ptr(bias), M, N, K,
        a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn), 1 if act == "gelu" else 0,
        int(accumulate), dt(a.dtype), dt(out.dtype), bn, split, sm_count(), ws.data_ptr(), ws.numel(),
        status_word().data_ptr(), stream(),
    )
    check(rc, "sb200_gemm_ws")
    return out


_FP8_FORMATS = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}


def gemm_fp8_supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    """True when ``gemm_fp8`` can multiply ``a [M, K]`` and ``b [N, K]`` on the fp8 tensor-core path."""
    return (a.is_cuda and a.dtype in _FP8_FORMATS and b.dtype in _FP8_FORMATS and a.dim() == 2 and b.dim() == 2
            and a.shape[1] == b.shape[1] and a.stride(1) == 1 and b.stride(1) == 1 and a.stride(0) % 16 == 0
            and b.stride(0) % 16 == 0 and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0
            and _lib.lib_has("sb200_gemm_fp8"))


def gemm_fp8(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None,
             out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``a [M, K] @ b [N, K]^T (+ bias)`` with fp8 (e4m3 / e5m2, mixed allowed) operands, unit scales, fp32
    accumulation in TMEM (``tcgen05.mma kind::f8f6f4``), result in bf16 or fp32."""
    assert gemm_fp8_supported(a, b), "gemm_fp8: operands must be row-major fp8 with rows of a multiple of 16 elements"
    assert out_dtype in (torch.bfloat16, torch.float32)
    M, Kd = a.shape
    N = b.shape[0]
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if bias is not None and (bias.dtype != torch.bfloat16 or not bias.is_contiguous()):
        bias = bias.to(torch.bfloat16).contiguous()
    ws = _gemm_workspace(a.device)
    check(lib().sb200_gemm_fp8(a.data_ptr(), b.data_ptr(), out.data_ptr(), ptr(bias), M, N, Kd, a.stride(0), b.stride(0),
                               out.stride(0), _FP8_FORMATS[a.dtype], _FP8_FORMATS[b.dtype], 0, dt(out_dtype), sm_count(),
                               ws.data_ptr(), ws.numel(), status_word().data_ptr(), stream()), "sb200_gemm_fp8")
    return out


_GEMM_WS: dict[int, torch.Tensor] = {}
_GEMM_WS_BYTES = 64 * 1024 * 1024


def _gemm_workspace(device: torch.device) -> torch.Tensor:
    """Split-K scratch of the GEMM (tile counters + fp32 partial tiles), one per device.  GEMMs that may run
    concurrently (issued on different streams without ordering between them) must not share it; the framework
    issues all its GEMMs on the current compute stream.  The kernel leaves the counters zero."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _GEMM_WS.get(key)
    if ws is None:
        ws = torch.zeros(_GEMM_WS_BYTES, dtype=torch.uint8, device=device)
        _GEMM_WS[key] = ws
    return ws


def _gemm_shape_exempt(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Shapes the TMA path cannot address (row pitch not a multiple of 16 bytes, unaligned views)."""
    return (
        a.dim() != 2
        or b.dim() != 2
        or a.stride(1) != 1
        or b.stride(1) != 1
        or a.stride(0) % 8 != 0
        or b.stride(0) % 8 != 0
        or a.data_ptr() % 16 != 0
        or b.data_ptr() % 16 != 0
        or a.shape[0] == 0
        or b.shape[0] == 0
        or a.shape[1] == 0
    )


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, act, wgrad):  # type: ignore[override]
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        pre = None
        if act == "gelu":
            pre = torch.empty((x2.shape[0], w.shape[0]), dtype=x.dtype, device=x.device)
        y = gemm(x2, w, bias=bias, act=act, pre_act_out=pre)
        ctx.save_for_backward(x2, w, pre)
        ctx.weight, ctx.bias = w, bias  # the parameter objects themselves (for their persistent .grad buffers)
        ctx.has_bias = bias is not None
        ctx.act = act
        ctx.wgrad = wgrad
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x2, w, pre = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        want_db = ctx.has_bias and ctx.needs_input_grad[2]
        bias_main = fused_grad_target(ctx.bias) if want_db else None
        bias_done = False
        if ctx.act == "gelu":
            fused = None
            if bias_main is not None and bias_main.dtype == dy2.dtype:
                # the bias gradient is the column sum of the GELU backward's output: one pass produces both
                fused = gelu_backward_with_bias_grad(dy2, pre, bias_main, accumulate=True)
            if fused is not None:
                dy2, bias_done = fused, True
            else:
                dy2 = gelu_backward(dy2, pre)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1] and ctx.wgrad:
            main = fused_grad_target(ctx.weight)
            if main is not None and main.dtype in (torch.float32, dy2.dtype):
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=True)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        if want_db and not bias_done:
            if bias_main is not None and bias_main.dtype == dy2.dtype:
                column_sum(dy2, out=bias_main, accumulate=True)
            else:
                db = column_sum(dy2)
        return dx, dw, db, None, None


def fused_grad_target(p: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """The persistent gradient buffer of a parameter that opted into in-kernel gradient accumulation.

    An optimizer that keeps ``param.grad`` as a permanent, zero-initialised view of a flat buffer sets
    ``param.fused_grad_accumulation = True``; backward kernels then add into ``param.grad`` from their epilogue and
    return no gradient for the parameter, which saves the separate accumulation pass per parameter.
    """
    if p is None or not getattr(p, "fused_grad_accumulation", False):
        return None
    g = p.grad
    if g is None or not g.is_contiguous() or g.shape != p.shape or not g.is_cuda:
        return None
    return g


def column_sum(x: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """Deterministic ``x[M, N].sum(0)`` (bias gradients); optionally added into ``out``."""
    M, N = x.shape
    if not (x.is_cuda and x.dtype in _KERNEL_DTYPES and x.stride(1) == 1 and N % (16 // x.element_size()) == 0
            and x.stride(0) % (16 // x.element_size()) == 0 and M > 0):
        r = x.sum(0)
        if out is None:
            return r
        return out.add_(r.to(out.dtype)) if accumulate else out.copy_(r)
    if out is None:
        out = torch.empty(N, dtype=x.dtype, device=x.device)
        accumulate = False
    assert out.dtype == x.dtype and out.is_contiguous()
    splits = lib().sb200_colsum_splits(M, N, x.element_size(), sm_count())
    partial = torch.empty((splits, N), dtype=torch.float32, device=x.device)
    check(lib().sb200_colsum(x.data_ptr(), out.data_ptr(), partial.data_ptr(), M, N, x.stride(0), splits,
                             int(accumulate), dt(x.dtype), stream()), "sb200_colsum")
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none") -> torch.Tensor:
    """``act(x @ w.T + bias)`` with the tcgen05 GEMM for forward, dgrad and wgrad on GPUs."""
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and w.dtype == x.dtype and _linear_ok(x, w):
        return _LinearFn.apply(x, w, bias, act, True)
    y = F.linear(x, w, bias)
    if act == "gelu":
        y = F.gelu(y)
    return y


def _linear_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    K = x.shape[-1]
    N = w.shape[0]
    return K % 8 == 0 and N % 8 == 0 and w.is_contiguous() and x.numel() > 0


# --------------------------------------------------------------------------- norms
class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps, rms):  # type: ignore[override]
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(M, dtype=torch.float32, device=x.device)
        mean = None if rms else torch.empty(M, dtype=torch.float32, device=x.device)
        wc = w if w.dtype == x.dtype else w.to(x.dtype)
        bc = None if b is None else (b if b.dtype == x.dtype else b.to(x.dtype))
        check(
            lib().sb200_norm_fwd(x2.data_ptr(), wc.data_ptr(), ptr(bc), y.data_ptr(), ptr(mean), rstd.data_ptr(),
                                 M, H, eps, int(rms), dt(x.dtype), stream()),
            "sb200_norm_fwd",
        )
        ctx.save_for_backward(x2, wc, mean, rstd)
        ctx.weight, ctx.bias = w, b
        ctx.rms = rms
        ctx.has_bias = b is not None
        ctx.w_dtype = w.dtype
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x2, w, mean, rstd = ctx.saved_tensors
        M, H = x2.shape
        dy2 = dy.reshape(M, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        rows = lib().sb200_norm_bwd_partial_rows_h(M, H, x2.element_size(), sm_count())
        dwp = torch.empty((rows, H), dtype=torch.float32, device=x2.device)
        dbp = torch.empty((rows, H), dtype=torch.float32, device=x2.device) if ctx.has_bias else None
        # parameters with a persistent gradient buffer of the compute dtype get their gradients added in place
        main_w = fused_grad_target(ctx.weight)
        main_b = fused_grad_target(ctx.bias) if ctx.has_bias else None
        fused = (main_w is not None and main_w.dtype == x2.dtype
                 and (not ctx.has_bias or (main_b is not None and main_b.dtype == x2.dtype)))
        if fused:
            dw, db = main_w, main_b
        else:
            dw = torch.empty(H, dtype=x2.dtype, device=x2.device)
            db = torch.empty(H, dtype=x2.dtype, device=x2.device) if ctx.has_bias else None
        check(
            lib().sb200_norm_bwd(dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), ptr(mean), rstd.data_ptr(),
                                 dx.data_ptr(), dwp.data_ptr(), ptr(dbp), dw.data_ptr(), ptr(db), M, H,
                                 int(ctx.rms), int(fused), rows, dt(x2.dtype), stream()),
            "sb200_norm_bwd",
        )
        if fused:
            return dx.view(dy.shape), None, None, None, None
        return dx.view(dy.shape), dw.to(ctx.w_dtype), (db.to(ctx.w_dtype) if db is not None else None), None, None


def _norm_kernel_ok(x: torch.Tensor) -> bool:
    if not x.is_cuda:
        return False
    if x.dtype not in _KERNEL_DTYPES:
        raise _lib.KernelError(f"norm: dtype {x.dtype} not supported on GPU")
    vec = 16 // x.element_size()
    H = x.shape[-1]
    return H % vec == 0 and H <= 256 * vec * 8 and x.numel() > 0


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if _norm_kernel_ok(x):
        return _NormFn.apply(x, weight, None, eps, True)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float = 1e-5) -> torch.Tensor:
    if _norm_kernel_ok(x):
        return _NormFn.apply(x, weight, bias, eps, False)
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


# --------------------------------------------------------------------------- activations
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, g, scale):  # type: ignore[override]
        F_ = a.shape[-1]
        a2, g2 = a.reshape(-1, F_), g.reshape(-1, F_)
        assert a2.stride(1) == 1 and g2.stride(1) == 1
        M = a2.shape[0]
        out = torch.empty((M, F_), dtype=a.dtype, device=a.device)
        check(
            lib().sb200_swiglu_fwd(a2.data_ptr(), g2.data_ptr(), out.data_ptr(), M, F_, a2.stride(0), g2.stride(0),
                                   F_, scale, dt(a.dtype), stream()),
            "sb200_swiglu_fwd",
        )
        ctx.save_for_backward(a2, g2)
        ctx.scale = scale
        ctx.shape = a.shape
        return out.view(a.shape)

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        a2, g2 = ctx.saved_tensors
        M, F_ = a2.shape
        d2 = dout.reshape(M, F_)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        da = torch.empty((M, F_), dtype=a2.dtype, device=a2.device)
        dg = torch.empty((M, F_), dtype=a2.dtype, device=a2.device)
        check(
            lib().sb200_swiglu_bwd(d2.data_ptr(), a2.data_ptr(), g2.data_ptr(), da.data_ptr(), dg.data_ptr(), M, F_,
                                   F_, a2.stride(0), g2.stride(0), F_, F_, ctx.scale, dt(a2.dtype), stream()),
            "sb200_swiglu_bwd",
        )
        return da.view(ctx.shape), dg.view(ctx.shape), None


def swiglu(a: torch.Tensor, g: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``silu(a) * g * scale``"""
    if a.is_cuda and a.dtype in _KERNEL_DTYPES:
        vec = 16 // a.element_size()
        a2, g2 = a.reshape(-1, a.shape[-1]), g.reshape(-1, g.shape[-1])
        if (a.shape[-1] % vec == 0 and a2.stride(-1) == 1 and g2.stride(-1) == 1 and a2.stride(0) % vec == 0
                and g2.stride(0) % vec == 0 and a.numel() > 0 and a2.data_ptr() % 16 == 0 and g2.data_ptr() % 16 == 0):
            return _SwiGLUFn.apply(a, g, float(scale))
    y = F.silu(a) * g
    return y if scale == 1.0 else y * scale


def gelu_backward(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    if dy.is_cuda and dy.dtype in _KERNEL_DTYPES and dy.is_contiguous() and x.is_contiguous():
        dx = torch.empty_like(dy)
        check(lib().sb200_gelu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), dy.numel(), dt(dy.dtype), stream()),
              "sb200_gelu_bwd")
        return dx
    xf = x.float()
    cdf = 0.5 * (1.0 + torch.erf(xf * 0.7071067811865476))
    pdf = torch.exp(-0.5 * xf * xf) * 0.3989422804014327
    return (dy.float() * (cdf + xf * pdf)).to(dy.dtype)


def gelu_backward_with_bias_grad(dy: torch.Tensor, x: torch.Tensor, bias_grad: torch.Tensor,
                                 accumulate: bool) -> Optional[torch.Tensor]:
    """``dx = dy * gelu'(x)`` and ``bias_grad (+)= dx.sum(0)`` in one pass over ``[M, N]`` tensors (the bias gradient of
    a linear layer with a fused GELU); returns None when the shapes do not fit the kernel (the caller then takes the
    two separate ops)."""
    M, N = dy.shape
    if not (dy.is_cuda and dy.dtype in _KERNEL_DTYPES and dy.is_contiguous() and x.is_contiguous() and x.shape == dy.shape
            and bias_grad.dtype == dy.dtype and bias_grad.is_contiguous() and N % (16 // dy.element_size()) == 0
            and _lib.lib_has("sb200_gelu_bwd_colsum")):
        return None
    dx = torch.empty_like(dy)
    splits = lib().sb200_colsum_splits(M, N, dy.element_size(), sm_count())
    partial = torch.empty((splits, N), dtype=torch.float32, device=dy.device)
    check(lib().sb200_gelu_bwd_colsum(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), bias_grad.data_ptr(),
                                      partial.data_ptr(), M, N, splits, int(accumulate), dt(dy.dtype), stream()),
          "sb200_gelu_bwd_colsum")
    return dx


class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):  # type: ignore[override]
        xc = x.contiguous()
        y = torch.empty_like(xc)
        check(lib().sb200_gelu_fwd(xc.data_ptr(), y.data_ptr(), xc.numel(), dt(x.dtype), stream()), "sb200_gelu_fwd")
        ctx.save_for_backward(xc)
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        (x,) = ctx.saved_tensors
        return gelu_backward(dy.contiguous(), x)


def gelu(x: torch.Tensor) -> torch.Tensor:
    if x.is_cuda and x.dtype in _KERNEL_DTYPES and x.numel() > 0:
        return _GeluFn.apply(x)
    return F.gelu(x)


# --------------------------------------------------------------------------- RoPE
def _rope_launch(x: torch.Tensor, pos: torch.Tensor, rot_dim: int, base: float, interleaved: bool, backward: bool):
    # x: [tokens, heads, d] with unit stride in d
    T, Hh, _ = x.shape
    check(
        lib().sb200_rope(x.data_ptr(), pos.data_ptr(), T, Hh, rot_dim, x.stride(0), x.stride(1), float(base),
                         int(interleaved), int(backward), dt(x.dtype), stream()),
        "sb200_rope",
    )


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos, rot_dim, base, interleaved):  # type: ignore[override]
        y = x.clone(memory_format=torch.contiguous_format)
        _rope_launch(y, pos, rot_dim, base, interleaved, False)
        ctx.save_for_backward(pos)
        ctx.args = (rot_dim, base, interleaved)
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        (pos,) = ctx.saved_tensors
        dx = dy.clone(memory_format=torch.contiguous_format)
        _rope_launch(dx, pos, *ctx.args, True)
        return dx, None, None, None, None


def rope_reference(x: torch.Tensor, pos: torch.Tensor, rot_dim: int, base: float, interleaved: bool) -> torch.Tensor:
    """Torch expression of the rotary embedding on ``x[tokens, heads, d]`` (fp32 angles)."""
    half = rot_dim // 2
    inv = torch.exp2(-math.log2(base) * (2.0 * torch.arange(half, device=x.device, dtype=torch.float32)) / rot_dim)
    ang = pos.to(torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    rot, rest = xf[..., :rot_dim], xf[..., rot_dim:]
    if interleaved:
        a, b = rot[..., 0::2], rot[..., 1::2]
        ra, rb = a * cos - b * sin, b * cos + a * sin
        out = torch.stack((ra, rb), dim=-1).flatten(-2)
    else:
        a, b = rot[..., :half], rot[..., half:]
        out = torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1)
    return torch.cat((out, rest), dim=-1).to(x.dtype)


def rope(x: torch.Tensor, pos: torch.Tensor, rot_dim: Optional[int] = None, base: float = 10000.0,
         interleaved: bool = False) -> torch.Tensor:
    """Rotary position embedding on ``x[tokens, heads, d]``; ``pos`` is ``[tokens]`` (any int dtype)."""
    rot_dim = rot_dim or x.shape[-1]
    if x.is_cuda and x.dtype in _KERNEL_DTYPES and x.numel() > 0:
        p32 = pos if pos.dtype == torch.int32 else pos.to(torch.int32)
        return _RopeFn.apply(x, p32.contiguous(), rot_dim, base, interleaved)
    return rope_reference(x, pos, rot_dim, base, interleaved)


# --------------------------------------------------------------------------- masked softmax
class _MaskedSoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, scale):  # type: ignore[override]
        b, h, sq, sk = x.shape
        xc = x.contiguous()
        y = torch.empty_like(xc)
        m8 = None
        if mask is not None:
            m8 = mask.expand(b, 1, sq, sk).contiguous().view(torch.uint8) if mask.dtype == torch.bool else mask
        check(
            lib().sb200_masked_softmax_fwd(xc.data_ptr(), ptr(m8), y.data_ptr(), b * h * sq, sk, h, sq, scale,
                                           dt(x.dtype), stream()),
            "sb200_masked_softmax_fwd",
        )
        ctx.save_for_backward(y, m8)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        y, m8 = ctx.saved_tensors
        b, h, sq, sk = y.shape
        dyc = dy.contiguous()
        dx = torch.empty_like(y)
        check(
            lib().sb200_masked_softmax_bwd(dyc.data_ptr(), y.data_ptr(), ptr(m8), dx.data_ptr(), b * h * sq, sk, h, sq,
                                           ctx.scale, dt(y.dtype), stream()),
            "sb200_masked_softmax_bwd",
        )
        return dx, None, None


def masked_softmax(x: torch.Tensor, mask: Optional[torch.Tensor], scale: float = 1.0,
                   softmax_in_fp32: bool = False) -> torch.Tensor:
    """``softmax(masked_fill(x * scale, mask, -10000))`` over the last dim of ``x[b, h, sq, sk]``.

    ``mask`` is boolean ``[b, 1, sq, sk]`` (broadcastable), True = masked out.
    """
    if x.is_cuda and x.dtype in _KERNEL_DTYPES and x.dim() == 4 and x.numel() > 0 and (
            mask is None or (mask.dim() == 4 and mask.shape[1] == 1)):
        return _MaskedSoftmaxFn.apply(x, mask, float(scale))
    in_dtype = x.dtype
    if softmax_in_fp32 and x.dtype != torch.float32:
        x = x.float()
    x = x * scale
    if mask is not None:
        x = x.masked_fill(mask, -10000.0)
    p = torch.softmax(x, dim=-1)
    return p.to(in_dtype)


# --------------------------------------------------------------------------- dropout + residual
def _launch_dropout_add(x: torch.Tensor, r: Optional[torch.Tensor], y: torch.Tensor, p: float, x_scale: float,
                        r_scale: float, rng: Optional[torch.Tensor], call: int, elem_offset: int, backward: bool) -> None:
    check(lib().sb200_dropout_add(x.data_ptr(), ptr(r), y.data_ptr(), x.numel(), p, x_scale, r_scale, ptr(rng), call,
                                  elem_offset, int(backward), dt(x.dtype), stream()), "sb200_dropout_add")


class _DropoutAddFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, p, x_scale, r_scale, rng, call, elem_offset, scale_grad):  # type: ignore[override]
        xc = x.contiguous()
        rc = None if residual is None else residual.contiguous()
        y = torch.empty_like(xc)
        _launch_dropout_add(xc, rc, y, p, x_scale, r_scale, rng, call, elem_offset, False)
        # scale_grad False: the scales act on the forward values only (unit-scaling's scale_fwd)
        ctx.args = (p, x_scale if scale_grad else 1.0, r_scale if scale_grad else 1.0, rng, call, elem_offset)
        ctx.has_residual = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        p, x_scale, r_scale, rng, call, elem_offset = ctx.args
        dyc = dy.contiguous()
        dx = dr = None
        if ctx.needs_input_grad[0]:
            if p == 0.0:
                dx = dyc if x_scale == 1.0 else dyc * x_scale
            else:
                dx = torch.empty_like(dyc)
                _launch_dropout_add(dyc, None, dx, p, x_scale, 0.0, rng, call, elem_offset, True)
        if ctx.has_residual and ctx.needs_input_grad[1]:
            dr = dyc if r_scale == 1.0 else dyc * r_scale
        return dx, dr, None, None, None, None, None, None, None


def dropout_add(x: torch.Tensor, residual: Optional[torch.Tensor], p: float, rng_state=None, training: bool = True,
                x_scale: float = 1.0, r_scale: float = 1.0, elem_offset: int = 0,
                scale_grad: bool = True) -> torch.Tensor:
    """``dropout(x, p) * x_scale + residual * r_scale`` in one pass (``residual`` may be None: plain dropout).

    ``rng_state`` is the ``KernelDropoutState`` of the topology: the mask depends on its seed and step (read on the
    device), on the index of this call inside the step and on the element's index ``elem_offset + i``, and is
    recomputed, not stored, for the backward pass.  On CPU tensors the torch expression is used."""
    p = float(p) if training else 0.0
    if p == 0.0 and residual is None:
        return x if x_scale == 1.0 else x * x_scale
    kernel = (x.is_cuda and x.dtype in _KERNEL_DTYPES and x.data_ptr() % 16 == 0 and elem_offset % 4 == 0
              and (residual is None or (residual.dtype == x.dtype and residual.shape == x.shape)))
    if kernel and p > 0.0 and rng_state is None:
        kernel = False
    if not kernel:
        from ..core.nn.scale import scale_fwd

        mul = (lambda t, s_: t * s_) if scale_grad else scale_fwd
        y = torch.nn.functional.dropout(x, p, training=True) if p > 0.0 else x
        if x_scale != 1.0:
            y = mul(y, x_scale)
        if residual is None:
            return y
        return y + (residual if r_scale == 1.0 else mul(residual, r_scale))
    rng, call = (rng_state.tensor(), rng_state.next_call()) if p > 0.0 else (None, 0)
    return _DropoutAddFn.apply(x, residual, p, float(x_scale), float(r_scale), rng, call, int(elem_offset), scale_grad)


def dropout_mask(shape: tuple, p: float, rng_state, call: int, dtype: torch.dtype = torch.float32,
                 elem_offset: int = 0) -> torch.Tensor:
    """The mask (values 0 or ``1 / (1 - p)``) that ``dropout_add`` applies for the given call index at the state's
    current step; for tests and debugging."""
    ones = torch.ones(shape, dtype=dtype, device=rng_state.device)
    out = torch.empty_like(ones)
    _launch_dropout_add(ones, None, out, p, 1.0, 0.0, rng_state.tensor(), call, elem_offset, False)
    return out


# --------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, W, vocab_start):  # type: ignore[override]
        idc = ids.reshape(-1).contiguous()
        T, H = idc.numel(), W.shape[1]
        out = torch.empty((T, H), dtype=W.dtype, device=W.device)
        check(
            lib().sb200_embedding_fwd(idc.data_ptr(), W.data_ptr(), out.data_ptr(), T, H, vocab_start, W.shape[0],
                                      dt(W.dtype), stream()),
            "sb200_embedding_fwd",
        )
        ctx.save_for_backward(idc)
        ctx.vocab_start = vocab_start
        ctx.w_shape = W.shape
        ctx.w_dtype = W.dtype
        return out.view(*ids.shape, H)

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        (idc,) = ctx.saved_tensors
        T = idc.numel()
        H = ctx.w_shape[1]
        d2 = dout.reshape(T, H).contiguous()
        sorted_ids, order = torch.sort(idc, stable=True)
        dW = torch.zeros(ctx.w_shape, dtype=torch.float32, device=dout.device)
        check(
            lib().sb200_embedding_bwd(sorted_ids.data_ptr(), order.data_ptr(), d2.data_ptr(), dW.data_ptr(), T, H,
                                      ctx.vocab_start, ctx.w_shape[0], dt(d2.dtype), dt(torch.float32), stream()),
            "sb200_embedding_bwd",
        )
        return None, dW.to(ctx.w_dtype), None


def embedding(ids: torch.Tensor, weight: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    """Rows of ``weight`` for ``ids - vocab_start``; ids outside ``[vocab_start, vocab_start + rows)`` give zeros."""
    if weight.is_cuda and weight.dtype in _KERNEL_DTYPES and ids.numel() > 0 and weight.is_contiguous():
        return _EmbeddingFn.apply(ids.to(torch.int64), weight, int(vocab_start))
    local = ids - vocab_start
    oob = (local < 0) | (local >= weight.shape[0])
    local = local.masked_fill(oob, 0)
    out = F.embedding(local, weight)
    return out.masked_fill(oob.unsqueeze(-1), 0.0)


# --------------------------------------------------------------------------- cross entropy
def ce_stats(logits: torch.Tensor, targets: torch.Tensor, vocab_start: int = 0, want_argmax: bool = True):
    """Per-token (max, sum exp(x-max), target logit or 0, argmax value, argmax index) over a vocab shard."""
    N, V = logits.shape
    if logits.is_cuda and logits.dtype in _KERNEL_DTYPES:
        assert logits.stride(1) == 1
        dev = logits.device
        rmax = torch.empty(N, dtype=torch.float32, device=dev)
        rsum = torch.empty(N, dtype=torch.float32, device=dev)
        tgt = torch.empty(N, dtype=torch.float32, device=dev)
        aval = torch.empty(N, dtype=torch.float32, device=dev) if want_argmax else None
        aidx = torch.empty(N, dtype=torch.int64, device=dev) if want_argmax else None
        tg = targets.reshape(-1).to(torch.int64).contiguous()
        check(
            lib().sb200_ce_stats(logits.data_ptr(), tg.data_ptr(), rmax.data_ptr(), rsum.data_ptr(), tgt.data_ptr(),
                                 ptr(aval), ptr(aidx), N, V, logits.stride(0), vocab_start, dt(logits.dtype),
                                 stream()),
            "sb200_ce_stats",
        )
        return rmax, rsum, tgt, aval, aidx
    lf = logits.float()
    rmax, aidx = lf.max(dim=-1)
    rsum = torch.exp(lf - rmax[:, None]).sum(-1)
    t = targets.reshape(-1).to(torch.int64) - vocab_start
    inside = (t >= 0) & (t < V)
    tgt = torch.where(inside, lf.gather(1, t.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(rmax))
    return rmax, rsum, tgt, rmax.clone(), aidx + vocab_start


def ce_finalize(logits: torch.Tensor, targets: torch.Tensor, gmax: torch.Tensor, gsum: torch.Tensor,
                gtgt: torch.Tensor, coef: Optional[torch.Tensor], vocab_start: int = 0, want_grad: bool = True,
                inplace: bool = True, scale_dev: Optional[torch.Tensor] = None):
    """Loss per token and (optionally) ``(softmax - onehot) * coef * scale_dev[0]`` written over the logits
    (``scale_dev``: a device scalar, e.g. the upstream gradient of the loss)."""
    N, V = logits.shape
    if logits.is_cuda and logits.dtype in _KERNEL_DTYPES:
        loss = torch.empty(N, dtype=torch.float32, device=logits.device)
        dl = None
        if want_grad:
            dl = logits if inplace else torch.empty_like(logits)
        tg = targets.reshape(-1).to(torch.int64).contiguous()
        check(
            lib().sb200_ce_finalize(logits.data_ptr(), tg.data_ptr(), gmax.data_ptr(), gsum.data_ptr(),
                                    gtgt.data_ptr(), ptr(coef), loss.data_ptr(), ptr(dl), N, V, logits.stride(0),
                                    dl.stride(0) if dl is not None else 0, vocab_start,
                                    ptr(None if scale_dev is None else scale_dev.reshape(-1)[:1].float().contiguous()),
                                    dt(logits.dtype), stream()),
            "sb200_ce_finalize",
        )
        return loss, dl
    lf = logits.float()
    loss = torch.log(gsum) + gmax - gtgt
    dl = None
    if want_grad:
        p = torch.exp(lf - gmax[:, None]) / gsum[:, None]
        t = targets.reshape(-1).to(torch.int64) - vocab_start
        inside = (t >= 0) & (t < V)
        onehot = torch.zeros_like(p)
        onehot[torch.arange(N, device=p.device)[inside], t[inside]] = 1.0
        p = p - onehot
        if coef is not None:
            p = p * coef[:, None]
        if scale_dev is not None:
            p = p * scale_dev.reshape(-1)[0].float()
        dl = p.to(logits.dtype)
    return loss, dl


def scale_by_device_scalar(x: torch.Tensor, scale_dev: Optional[torch.Tensor], scale: float = 1.0) -> torch.Tensor:
    """In place ``x *= scale * scale_dev[0]`` without a host sync."""
    if x.is_cuda and x.dtype in _KERNEL_DTYPES and x.is_contiguous():
        sd = None
        if scale_dev is not None:
            sd = scale_dev.reshape(-1)[:1].to(torch.float32)
        check(lib().sb200_scale_by_dev(x.data_ptr(), ptr(sd), scale, x.numel(), dt(x.dtype), stream()),
              "sb200_scale_by_dev")
        return x
    s = scale if scale_dev is None else scale_dev.reshape(-1)[0].to(torch.float32) * scale
    return x.mul_(s)


# --------------------------------------------------------------------------- optimizer kernels
def adamw_step(p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor, p_lp: Optional[torch.Tensor],
               lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
               control: Optional[torch.Tensor] = None, hyper: Optional[torch.Tensor] = None) -> None:
    """Fused AdamW on flat fp32 ``p, m, v`` with gradient ``g`` (any float dtype) and optional low-precision copy.

    ``control`` is a device float[2]: gradient multiplier and a skip flag (non-zero = leave everything untouched).
    ``hyper`` is an optional device float[3] ``[lr, 1 - beta1^t, 1 - beta2^t]`` that overrides ``lr`` and ``step``
    (so that a captured CUDA graph can be replayed with new values).
    """
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if p.is_cuda:
        assert p.dtype == torch.float32 and p.is_contiguous() and g.is_contiguous()
        check(
            lib().sb200_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), ptr(p_lp), p.numel(), lr, beta1,
                              beta2, eps, weight_decay, bc1, bc2, ptr(control), ptr(hyper), dt(g.dtype),
                              dt(p_lp.dtype) if p_lp is not None else 0, stream()),
            "sb200_adamw",
        )
        return
    if hyper is not None:
        lr, bc1, bc2 = (float(v) for v in hyper.tolist())
    gmul = 1.0
    if control is not None:
        if float(control[1]) != 0.0:
            return
        gmul = float(control[0])
    gf = g if g.dtype == torch.float32 else g.float()
    if gmul != 1.0:
        gf = gf * gmul
    p.mul_(1.0 - lr * weight_decay)
    m.mul_(beta1).add_(gf, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1.0 - beta2)
    denom = v.sqrt().div_(math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
    if p_lp is not None:
        p_lp.copy_(p)


_SUMSQ_SCRATCH: dict[int, torch.Tensor] = {}


def sumsq_(g: torch.Tensor, out: torch.Tensor, flag: Optional[torch.Tensor], scale: float = 1.0,
           accumulate: bool = True) -> None:
    """``out[0] (+)= scale * sum(g^2)`` and ``flag[0] = 1`` if ``g`` holds inf/nan — no host sync."""
    if g.is_cuda:
        d = g.device.index
        if d not in _SUMSQ_SCRATCH:
            _SUMSQ_SCRATCH[d] = torch.empty(lib().sb200_sumsq_max_partials(), dtype=torch.float32, device=g.device)
        gc = g if g.is_contiguous() else g.contiguous()
        check(
            lib().sb200_sumsq(gc.data_ptr(), gc.numel(), _SUMSQ_SCRATCH[d].data_ptr(), out.data_ptr(), ptr(flag),
                              scale, int(accumulate), dt(g.dtype), stream()),
            "sb200_sumsq",
        )
        return
    gf = g.reshape(-1) if g.dtype == torch.float32 else g.reshape(-1).float()
    raw = torch.dot(gf, gf)  # no squared copy; inf / nan anywhere in g makes the sum non-finite
    s = raw * scale
    if accumulate:
        out[0] += s
    else:
        out[0] = s
    if flag is not None and not bool(torch.isfinite(raw)):
        flag[0] = 1


def step_control(which: int, stats: torch.Tensor, flag: torch.Tensor, control: torch.Tensor, result: torch.Tensor,
                 inv: float = 1.0, clip: float = 0.0, replicas: float = 1.0) -> None:
    """Scalar bookkeeping of an optimizer step on the device, one launch each, no host synchronisation.

    ``which`` 0: ``stats[1:3] = [overflow flag, device status word]`` (before the statistics are summed over the
    ranks); 1: from the summed ``stats`` derive ``control = [gradient multiplier, skip]`` and ``result = [global
    norm, skip, a device-side wait gave up, norm after clipping]``; 2: fold a status raised after that into
    ``result[2]``."""
    if stats.is_cuda:
        check(lib().sb200_step_control(which, stats.data_ptr(), flag.data_ptr(), status_word().data_ptr(), inv, clip,
                                       replicas, control.data_ptr(), result.data_ptr(), stream()), "sb200_step_control")
        return
    if which == 0:
        stats[1] = float(flag[0] != 0)
        stats[2] = 0.0
    elif which == 1:
        norm = math.sqrt(float(stats[0]) / replicas) * inv if float(stats[0]) >= 0 else float("nan")
        timed_out = float(stats[2]) > 0
        bad = float(stats[1]) > 0 or not math.isfinite(norm) or timed_out
        coef = clip / norm if (clip > 0.0 and norm >= clip) else 1.0
        control[0] = 0.0 if bad else coef * inv
        control[1] = float(bad)
        result[0] = norm
        result[1] = float(bad)
        result[2] = float(timed_out)
        result[3] = norm * coef


def transpose2d(x: torch.Tensor) -> torch.Tensor:
    if x.is_cuda and x.dtype in _KERNEL_DTYPES and x.is_contiguous() and x.dim() == 2:
        out = torch.empty((x.shape[1], x.shape[0]), dtype=x.dtype, device=x.device)
        check(lib().sb200_transpose(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], dt(x.dtype), stream()),
              "sb200_transpose")
        return out
    return x.t().contiguous()
