"""Autograd wrapper of the tcgen05 flash-attention kernels (``sb200_fa_fwd`` / ``sb200_fa_bwd``)."""

from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from . import _lib
from ._lib import check, lib, stream
from .functional import status_word

_DECLARED = False


def _declare() -> None:
    global _DECLARED
    if _DECLARED:
        return
    _lib.declare("sb200_fa_fwd", [c_void_p] * 7 + [c_int] * 4 + [c_long, c_int, c_long, c_int, c_long, c_int, c_int,
                                                                 c_int, c_float, c_void_p, c_void_p])
    _lib.declare("sb200_fa_bwd_splits", [c_int] * 4)
    _lib.declare("sb200_fa_bwd", [c_void_p] * 8 + [c_int] + [c_void_p] * 5 + [c_int] * 4 + [c_long, c_int, c_long, c_int, c_long, c_int, c_int,
                                                                  c_int, c_float, c_void_p, c_void_p])
    _lib.declare("sb200_fa_bwd_strided", [c_void_p] * 8 + [c_int] + [c_void_p] * 5 + [c_int] * 4
                 + [c_long, c_int] * 6 + [c_int, c_int, c_float, c_void_p, c_void_p])
    _lib.declare("sb200_rope_multi", [c_void_p, c_void_p, c_int, c_int, c_int, c_long, c_long, c_int, c_long, c_float,
                                      c_int, c_int, c_int, c_void_p])
    _DECLARED = True


_DOC_CACHE: dict[str, tuple] = {}


def doc_ranges(cu_seqlens: torch.Tensor, total: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Per token: first token index of its document and one past its last (int32, cached per cu_seqlens tensor)."""
    key = (cu_seqlens.data_ptr(), cu_seqlens._version, total, cu_seqlens.numel())
    hit = _DOC_CACHE.get("last")
    if hit is not None and hit[0] == key:
        return hit[1], hit[2]
    cu = cu_seqlens.to(torch.int64)
    idx = torch.arange(total, device=cu.device)
    doc = (torch.searchsorted(cu, idx, right=True) - 1).clamp_(0, cu.numel() - 2)
    start = cu[doc].to(torch.int32).contiguous()
    end = cu[doc + 1].to(torch.int32).contiguous()
    _DOC_CACHE["last"] = (key, start, end, cu_seqlens)  # keep cu_seqlens alive so the pointer stays unique
    return start, end


def _check_ranges(start: torch.Tensor, end: torch.Tensor, tokens: int) -> None:
    # the kernels read one (start, end) pair per token
    if start.numel() != tokens or end.numel() != tokens or start.dtype != torch.int32 or end.dtype != torch.int32:
        raise ValueError(f"document ranges cover {start.numel()} / {end.numel()} tokens ({start.dtype}), "
                         f"attention runs on {tokens}")


def _strides_ok(t: torch.Tensor) -> bool:
    return t.stride(2) == 1 and t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0


def _prep(t: torch.Tensor) -> torch.Tensor:
    return t if _strides_ok(t) else t.contiguous()


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, doc_start, doc_end, causal, scale, window):  # type: ignore[override]
        _declare()
        q, k, v = _prep(q), _prep(k), _prep(v)
        T, Hq, D = q.shape
        Hkv = k.shape[1]
        o = torch.empty((T, Hq, D), dtype=q.dtype, device=q.device)
        lse2 = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
        check(
            lib().sb200_fa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse2.data_ptr(),
                               doc_start.data_ptr(), doc_end.data_ptr(), T, Hq, Hkv, D, q.stride(0), q.stride(1),
                               k.stride(0), k.stride(1), v.stride(0), v.stride(1), int(causal),
                               -1 if window is None else int(window), float(scale), status_word().data_ptr(), stream()),
            "sb200_fa_fwd",
        )
        ctx.save_for_backward(q, k, v, o, lse2, doc_start, doc_end)
        ctx.cfg = (causal, scale, window)
        return o

    @staticmethod
    def backward(ctx, do):  # type: ignore[override]
        q, k, v, o, lse2, doc_start, doc_end = ctx.saved_tensors
        causal, scale, window = ctx.cfg
        T, Hq, D = q.shape
        Hkv = k.shape[1]
        do = do.contiguous()
        dq = torch.empty((T, Hq, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((T, Hkv, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((T, Hkv, D), dtype=q.dtype, device=q.device)
        delta = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
        splits = lib()._handle.sb200_fa_bwd_splits(T, Hq, Hkv, _lib.sm_count())
        partial = None
        if splits > 1:
            partial = torch.empty((2, splits, T, Hkv, D), dtype=torch.float32, device=q.device)
        check(
            lib().sb200_fa_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse2.data_ptr(),
                               delta.data_ptr(), _lib.ptr(partial), splits, dq.data_ptr(), dk.data_ptr(),
                               dv.data_ptr(), doc_start.data_ptr(),
                               doc_end.data_ptr(), T, Hq, Hkv, D, q.stride(0), q.stride(1), k.stride(0), k.stride(1),
                               v.stride(0), v.stride(1), int(causal), -1 if window is None else int(window),
                               float(scale), status_word().data_ptr(), stream()),
            "sb200_fa_bwd",
        )
        return dq, dk, dv, None, None, None, None, None


def flash_attention_kernel(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: Optional[torch.Tensor],
                           causal: bool, scale: float, window: Optional[int],
                           ranges: Optional[tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
    if q.dtype != torch.bfloat16:
        # the kernels are bf16; fp16 inputs are converted (same exponent-safe range for attention inputs)
        out = flash_attention_kernel(q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16), cu_seqlens,
                                     causal, scale, window, ranges)
        return out.to(q.dtype)
    start, end = ranges if ranges is not None else doc_ranges(cu_seqlens, q.shape[0])
    _check_ranges(start, end, q.shape[0])
    return _FlashAttention.apply(q, k, v, start, end, causal, scale, window)


class _PackedQKVAttention(torch.autograd.Function):
    """Self-attention on a packed projection ``qkv[T, heads, 3 * d]`` (per head ``[q | k | v]``).

    The rotary embedding is applied in place on the q and k parts, the attention kernels read q, k and v as strided
    views, and the backward pass writes dq, dk and dv straight into one ``[T, heads, 3 * d]`` gradient (followed by
    the inverse rotation in place) - no slicing, concatenation or copies on either pass.  ``qkv`` is consumed: its
    contents are the rotated projection afterwards.
    """

    @staticmethod
    def forward(ctx, qkv, pos, rot, doc_start, doc_end, causal, scale, window):  # type: ignore[override]
        _declare()
        T, H, D3 = qkv.shape
        D = D3 // 3
        assert qkv.is_contiguous() and qkv.dtype == torch.bfloat16
        if rot is not None:
            rot_dim, base, interleaved = rot
            check(lib().sb200_rope_multi(qkv.data_ptr(), pos.data_ptr(), T, H, rot_dim, H * D3, D3, 2, D, float(base),
                                         int(interleaved), 0, _lib.dt(qkv.dtype), stream()), "sb200_rope_multi")
        q, k, v = qkv[..., :D], qkv[..., D:2 * D], qkv[..., 2 * D:]
        o = torch.empty((T, H, D), dtype=qkv.dtype, device=qkv.device)
        lse2 = torch.empty((H, T), dtype=torch.float32, device=qkv.device)
        check(
            lib().sb200_fa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse2.data_ptr(),
                               doc_start.data_ptr(), doc_end.data_ptr(), T, H, H, D, H * D3, D3, H * D3, D3, H * D3, D3,
                               int(causal), -1 if window is None else int(window), float(scale),
                               status_word().data_ptr(), stream()),
            "sb200_fa_fwd",
        )
        ctx.save_for_backward(qkv, o, lse2, doc_start, doc_end, pos if rot is not None else None)
        ctx.cfg = (causal, scale, window, rot)
        return o

    @staticmethod
    def backward(ctx, do):  # type: ignore[override]
        qkv, o, lse2, doc_start, doc_end, pos = ctx.saved_tensors
        causal, scale, window, rot = ctx.cfg
        T, H, D3 = qkv.shape
        D = D3 // 3
        do = do.contiguous()
        q, k, v = qkv[..., :D], qkv[..., D:2 * D], qkv[..., 2 * D:]
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[..., :D], dqkv[..., D:2 * D], dqkv[..., 2 * D:]
        delta = torch.empty((H, T), dtype=torch.float32, device=qkv.device)
        splits = lib()._handle.sb200_fa_bwd_splits(T, H, H, _lib.sm_count())
        partial = None
        if splits > 1:
            partial = torch.empty((2, splits, T, H, D), dtype=torch.float32, device=qkv.device)
        ld = (H * D3, D3)
        check(
            lib().sb200_fa_bwd_strided(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(),
                                       lse2.data_ptr(), delta.data_ptr(), _lib.ptr(partial), splits, dq.data_ptr(),
                                       dk.data_ptr(), dv.data_ptr(), doc_start.data_ptr(), doc_end.data_ptr(), T, H, H,
                                       D, *ld, *ld, *ld, *ld, *ld, *ld, int(causal),
                                       -1 if window is None else int(window), float(scale),
                                       status_word().data_ptr(), stream()),
            "sb200_fa_bwd_strided",
        )
        if rot is not None:
            rot_dim, base, interleaved = rot
            check(lib().sb200_rope_multi(dqkv.data_ptr(), pos.data_ptr(), T, H, rot_dim, H * D3, D3, 2, D, float(base),
                                         int(interleaved), 1, _lib.dt(dqkv.dtype), stream()), "sb200_rope_multi")
        return dqkv, None, None, None, None, None, None, None


def packed_qkv_supported(qkv: torch.Tensor) -> bool:
    """True when ``packed_qkv_attention`` can run on ``qkv[T, heads, 3 * d]``."""
    return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 3 and qkv.shape[-1] % 3 == 0
            and qkv.shape[-1] // 3 in (64, 128) and qkv.is_contiguous() and _lib.lib_has("sb200_fa_bwd_strided"))


def packed_qkv_attention(qkv: torch.Tensor, positions: Optional[torch.Tensor],
                         rotary: Optional[tuple[int, float, bool]], cu_seqlens: Optional[torch.Tensor], causal: bool,
                         scale: float, window: Optional[int],
                         ranges: Optional[tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
    """Rotary embedding + self-attention on a packed projection; returns ``[T, heads, d]``.

    ``rotary = (rotary dimensions, base, interleaved)`` or None; ``positions`` is ``[T]``.  ``qkv`` is overwritten
    with the rotated projection.
    """
    start, end = ranges if ranges is not None else doc_ranges(cu_seqlens, qkv.shape[0])
    _check_ranges(start, end, qkv.shape[0])
    pos = None
    if rotary is not None:
        assert positions is not None
        pos = positions if positions.dtype == torch.int32 else positions.to(torch.int32)
        pos = pos.contiguous()
    return _PackedQKVAttention.apply(qkv, pos, rotary, start, end, causal, scale, window)
