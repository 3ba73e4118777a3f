"""Autograd wrapper of the tcgen05 flash-attention kernels (``sb200_fa_fwd`` / ``sb200_fa_bwd``)."""

from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_uint, c_void_p
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
    # dropout probability, device {seed, step}, call index, first head; then the element type (SB_DT_BF16 / SB_DT_F16)
    drop = [c_float, c_void_p, c_uint, c_int, c_int]
    _lib.declare("sb200_fa_fwd", [c_void_p] * 7 + [c_int] * 4 + [c_long, c_int, c_long, c_int, c_long, c_int, c_int,
                                                                 c_int, c_float] + drop + [c_void_p, c_void_p])
    _lib.declare("sb200_fa_bwd_splits", [c_int] * 4)
    _lib.declare("sb200_fa_bwd", [c_void_p] * 8 + [c_int] + [c_void_p] * 5 + [c_int] * 4 + [c_long, c_int, c_long, c_int, c_long, c_int, c_int,
                                                                  c_int, c_float] + drop + [c_void_p, c_void_p])
    _lib.declare("sb200_fa_bwd_strided", [c_void_p] * 8 + [c_int] + [c_void_p] * 5 + [c_int] * 4
                 + [c_long, c_int] * 6 + [c_int, c_int, c_float] + drop + [c_void_p, c_void_p])
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
    def forward(ctx, q, k, v, doc_start, doc_end, causal, scale, window, drop):  # type: ignore[override]
        _declare()
        q, k, v = _prep(q), _prep(k), _prep(v)
        dp, drng, dcall, dhead = drop
        T, Hq, D = q.shape
        Hkv = k.shape[1]
        o = torch.empty((T, Hq, D), dtype=q.dtype, device=q.device)
        lse2 = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
        check(
            lib().sb200_fa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse2.data_ptr(),
                               doc_start.data_ptr(), doc_end.data_ptr(), T, Hq, Hkv, D, q.stride(0), q.stride(1),
                               k.stride(0), k.stride(1), v.stride(0), v.stride(1), int(causal),
                               -1 if window is None else int(window), float(scale), dp, _lib.ptr(drng), dcall, dhead,
                               _lib.dt(q.dtype), status_word().data_ptr(), stream()),
            "sb200_fa_fwd",
        )
        ctx.save_for_backward(q, k, v, o, lse2, doc_start, doc_end)
        ctx.cfg = (causal, scale, window, drop)
        return o

    @staticmethod
    def backward(ctx, do):  # type: ignore[override]
        q, k, v, o, lse2, doc_start, doc_end = ctx.saved_tensors
        causal, scale, window, (dp, drng, dcall, dhead) = ctx.cfg
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
                               float(scale), dp, _lib.ptr(drng), dcall, dhead, _lib.dt(q.dtype),
                               status_word().data_ptr(), stream()),
            "sb200_fa_bwd",
        )
        return dq, dk, dv, None, None, None, None, None, None


NO_DROPOUT = (0.0, None, 0, 0)


def dropout_args(dropout_p: float, rng_state, head_offset: int = 0) -> tuple:
    """(probability, device {seed, step}, call index, first head) for one attention call; draws the next call index
    of the ``KernelDropoutState``.  ``head_offset`` is the index of this rank's first head among all heads of the layer
    (tensor-parallel ranks share seed and call index and differ in their heads).  The kernels quantise the
    probability to a multiple of 1/256."""
    if dropout_p <= 0.0:
        return NO_DROPOUT
    assert rng_state is not None, "attention dropout in the kernel needs the topology's KernelDropoutState"
    return (float(dropout_p), rng_state.tensor(), rng_state.next_call(), int(head_offset))


def flash_attention_kernel(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: Optional[torch.Tensor],
                           causal: bool, scale: float, window: Optional[int],
                           ranges: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
                           drop: tuple = NO_DROPOUT) -> torch.Tensor:
    assert q.dtype in (torch.bfloat16, torch.float16) and k.dtype == q.dtype and v.dtype == q.dtype, (
        f"the attention kernels take bf16 or fp16 tensors of one type, got {q.dtype}, {k.dtype}, {v.dtype}")
    start, end = ranges if ranges is not None else doc_ranges(cu_seqlens, q.shape[0])
    _check_ranges(start, end, q.shape[0])
    return _FlashAttention.apply(q, k, v, start, end, causal, scale, window, drop)


def attention_dropout_mask(T: int, heads: int, dropout_p: float, rng_state, call: int) -> torch.Tensor:
    """The mask ``[heads, T, T]`` (0 or ``1 / (1 - p)`` with p quantised to 1/256) that the attention kernels apply
    for the given call index at the state's current step, obtained by running the forward kernel on inputs that make
    every allowed probability equal (q = 0) and reading the result through one-hot values; for tests."""
    dev = rng_state.device
    out = torch.zeros((heads, T, T), dtype=torch.float32, device=dev)
    q = torch.zeros((T, heads, 64), dtype=torch.bfloat16, device=dev)
    start = torch.zeros(T, dtype=torch.int32, device=dev)
    end = torch.full((T,), T, dtype=torch.int32, device=dev)
    for c0 in range(0, T, 64):  # 64 one-hot value columns at a time: o[t, h, j] = mask[h, t, c0 + j] / T
        v = torch.zeros((T, heads, 64), dtype=torch.bfloat16, device=dev)
        n = min(64, T - c0)
        v[torch.arange(c0, c0 + n, device=dev), :, torch.arange(n, device=dev)] = 1.0
        o = _FlashAttention.apply(q, q, v, start, end, False, 1.0, None, (float(dropout_p), rng_state.tensor(), call, 0))
        out[:, :, c0:c0 + n] = (o.float() * T).permute(1, 0, 2)[:, :, :n]
    return out


class _PackedQKVAttention(torch.autograd.Function):
    """Self-attention on a packed projection ``qkv[T, heads, 3 * d]`` (per head ``[q | k | v]``).

    The rotary embedding is applied in place on the q and k parts, the attention kernels read q, k and v as strided
    views, and the backward pass writes dq, dk and dv straight into one ``[T, heads, 3 * d]`` gradient (followed by
    the inverse rotation in place) - no slicing, concatenation or copies on either pass.  ``qkv`` is consumed: its
    contents are the rotated projection afterwards.
    """

    @staticmethod
    def forward(ctx, qkv, pos, rot, doc_start, doc_end, causal, scale, window, drop):  # type: ignore[override]
        _declare()
        dp, drng, dcall, dhead = drop
        T, H, D3 = qkv.shape
        D = D3 // 3
        assert qkv.is_contiguous() and qkv.dtype in (torch.bfloat16, torch.float16)
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
                               int(causal), -1 if window is None else int(window), float(scale), dp, _lib.ptr(drng),
                               dcall, dhead, _lib.dt(qkv.dtype), status_word().data_ptr(), stream()),
            "sb200_fa_fwd",
        )
        ctx.save_for_backward(qkv, o, lse2, doc_start, doc_end, pos if rot is not None else None)
        ctx.cfg = (causal, scale, window, rot, drop)
        return o

    @staticmethod
    def backward(ctx, do):  # type: ignore[override]
        qkv, o, lse2, doc_start, doc_end, pos = ctx.saved_tensors
        causal, scale, window, rot, (dp, drng, dcall, dhead) = ctx.cfg
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
                                       -1 if window is None else int(window), float(scale), dp, _lib.ptr(drng),
                                       dcall, dhead, _lib.dt(qkv.dtype), status_word().data_ptr(), stream()),
            "sb200_fa_bwd_strided",
        )
        if rot is not None:
            rot_dim, base, interleaved = rot
            check(lib().sb200_rope_multi(dqkv.data_ptr(), pos.data_ptr(), T, H, rot_dim, H * D3, D3, 2, D, float(base),
                                         int(interleaved), 1, _lib.dt(dqkv.dtype), stream()), "sb200_rope_multi")
        return dqkv, None, None, None, None, None, None, None, None


def packed_qkv_supported(qkv: torch.Tensor) -> bool:
    """True when ``packed_qkv_attention`` can run on ``qkv[T, heads, 3 * d]``."""
    return (qkv.is_cuda and qkv.dtype in (torch.bfloat16, torch.float16) and qkv.dim() == 3 and qkv.shape[-1] % 3 == 0
            and qkv.shape[-1] // 3 in (64, 128) and qkv.is_contiguous() and _lib.lib_has("sb200_fa_bwd_strided"))


def packed_qkv_attention(qkv: torch.Tensor, positions: Optional[torch.Tensor],
                         rotary: Optional[tuple[int, float, bool]], cu_seqlens: Optional[torch.Tensor], causal: bool,
                         scale: float, window: Optional[int],
                         ranges: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
                         drop: tuple = NO_DROPOUT) -> torch.Tensor:
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
    return _PackedQKVAttention.apply(qkv, pos, rotary, start, end, causal, scale, window, drop)


# ------------------------------------------------------------------------------------------ cross-length attention
def key_ranges(cu_q: torch.Tensor, cu_k: torch.Tensor, tq: int, causal: bool,
               window: Optional[int]) -> tuple[torch.Tensor, torch.Tensor]:
    """For every packed query token the half-open range of packed key indices it may attend to (int32 ``[tq]`` each):
    the keys of its own document, up to the causal diagonal (aligned to the end of the keys, so the last query sees
    every key) and inside the local window.  Built with tensor operations only: no host synchronisation."""
    cq, ck = cu_q.to(torch.int64), cu_k.to(torch.int64)
    idx = torch.arange(tq, device=cq.device)
    doc = (torch.searchsorted(cq, idx, right=True) - 1).clamp_(0, cq.numel() - 2)
    len_q, len_k = (cq[1:] - cq[:-1])[doc], (ck[1:] - ck[:-1])[doc]
    centre = idx - cq[doc] + (len_k - len_q)  # key position on the diagonal of this query
    lo = torch.zeros_like(centre)
    hi = len_k.clone()
    if causal:
        hi = torch.minimum(hi, centre + 1)
    if window is not None and window >= 0:
        lo = torch.maximum(lo, centre - window)
        if not causal:
            hi = torch.minimum(hi, centre + window + 1)
    lo = lo.clamp_(min=0)
    hi = torch.maximum(hi, lo)
    base = ck[doc]
    return (base + lo).to(torch.int32).contiguous(), (base + hi).to(torch.int32).contiguous()


def decode_supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    return (q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and q.shape[-1] in (64, 128)
            and q.shape[1] % k.shape[1] == 0 and k.shape == v.shape and _lib.lib_has("sb200_fa_decode")
            and not (torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)))


def flash_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_q: torch.Tensor, cu_k: torch.Tensor,
                 causal: bool, scale: float, window: Optional[int]) -> torch.Tensor:
    """Queries and keys of different lengths (decoding against a KV cache): ``q [Tq, Hq, D]``, ``k / v [Tk, Hkv, D]``.
    Forward only."""
    _lib.declare("sb200_fa_decode", [c_void_p] * 6 + [c_int] * 4 + [c_long] * 8 + [c_float, c_int, c_void_p])
    q = q if q.stride(2) == 1 else q.contiguous()
    k = k if _strides_ok(k) else k.contiguous()
    v = v if _strides_ok(v) else v.contiguous()
    lo, hi = key_ranges(cu_q, cu_k, q.shape[0], causal, window)
    hi.clamp_(max=k.shape[0])  # cumulative lengths that overshoot the key tensor must not become addresses
    out = torch.empty_like(q, memory_format=torch.contiguous_format)
    check(
        lib().sb200_fa_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lo.data_ptr(), hi.data_ptr(),
                              q.shape[0], q.shape[1], k.shape[1], q.shape[2], q.stride(0), q.stride(1), k.stride(0),
                              k.stride(1), v.stride(0), v.stride(1), out.stride(0), out.stride(1), float(scale),
                              _lib.dt(q.dtype), stream()),
        "sb200_fa_decode",
    )
    return out
