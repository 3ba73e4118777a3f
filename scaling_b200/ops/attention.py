"""Variable-length (packed) multi-head attention with MQA/GQA, causal masking and local windows.

``flash_attention`` takes token-major tensors ``q[Tq, Hq, D]``, ``k/v[Tk, Hkv, D]`` and cumulative
sequence lengths (int32, ``[n_docs + 1]``), like the call the reference makes into the flash-attn
package (src/scaling/core/nn/attention/attention.py:216-271).  On GPUs with bf16/fp16 inputs and
``D in {64, 128}`` the hand-written tcgen05 kernels run (forward and deterministic backward; smaller head
sizes are padded to these), and queries against a longer KV cache go to a streaming decode kernel; the
dense torch expression below serves CPU ranks and head sizes above 128, and is the numerical oracle of
the kernel tests.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from . import _lib


def _doc_ids(cu: torch.Tensor, total: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(document index, position inside the document) for each of ``total`` packed tokens."""
    idx = torch.arange(total, device=cu.device)
    doc = torch.searchsorted(cu.to(torch.int64), idx, right=True) - 1
    doc = doc.clamp_(0, cu.numel() - 2)
    pos = idx - cu.to(torch.int64)[doc]
    return doc, pos


def attention_mask_from_cu_seqlens(cu_q: torch.Tensor, cu_k: torch.Tensor, tq: int, tk: int, causal: bool,
                                   window: Optional[int]) -> torch.Tensor:
    """Boolean ``[tq, tk]`` matrix, True where a query may attend to a key."""
    dq, pq = _doc_ids(cu_q, tq)
    dk, pk = _doc_ids(cu_k, tk)
    allowed = dq[:, None] == dk[None, :]
    len_q = (cu_q[1:] - cu_q[:-1]).to(torch.int64)[dq]
    len_k = (cu_k[1:] - cu_k[:-1]).to(torch.int64)[dq]
    shift = (len_k - len_q)[:, None]  # causal diagonal is aligned to the end of the keys
    rel = pk[None, :] - (pq[:, None] + shift)
    if causal:
        allowed &= rel <= 0
    if window is not None and window >= 0:
        allowed &= rel >= -window
        if not causal:
            allowed &= rel <= window
    return allowed


def attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_q: torch.Tensor,
                        cu_k: Optional[torch.Tensor], causal: bool, scale: float,
                        window: Optional[int] = None, dropout_p: float = 0.0,
                        dropout_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dense O(T^2) evaluation in fp32; returns ``[Tq, Hq, D]`` in the dtype of ``q``.  ``dropout_mask``
    (``[Hq, Tq, Tk]``, entries 0 or ``1 / (1 - p)``) replaces the random draw of ``dropout_p``."""
    cu_k = cu_q if cu_k is None else cu_k
    tq, hq, d = q.shape
    tk, hkv, _ = k.shape
    rep = hq // hkv
    qf = q.float().transpose(0, 1)  # [Hq, Tq, D]
    kf = k.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    vf = v.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    scores = torch.matmul(qf, kf.transpose(1, 2)) * scale
    allowed = attention_mask_from_cu_seqlens(cu_q, cu_k, tq, tk, causal, window)
    scores = scores.masked_fill(~allowed[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    probs = torch.nan_to_num(probs, nan=0.0)  # fully masked rows
    if dropout_mask is not None:
        probs = probs * dropout_mask.to(probs.dtype)
    elif dropout_p > 0.0:
        probs = torch.nn.functional.dropout(probs, dropout_p)
    out = torch.matmul(probs, vf)
    return out.transpose(0, 1).to(q.dtype)


def _uniform_docs(cu: torch.Tensor, total: int) -> Optional[int]:
    """Length L if the packed batch consists of total/L documents of equal length L, else None."""
    n = cu.numel() - 1
    if n <= 0 or total % n != 0:
        return None
    L = total // n
    expect = torch.arange(0, total + 1, L, device=cu.device, dtype=cu.dtype)
    return L if expect.numel() == cu.numel() and bool(torch.equal(expect, cu)) else None


def kernel_supported(q: torch.Tensor, k: torch.Tensor, cu_k: Optional[torch.Tensor]) -> bool:
    return (
        q.is_cuda
        and q.dtype in (torch.bfloat16, torch.float16)
        and q.shape[-1] in (64, 128)
        and cu_k is None
        and q.shape[0] == k.shape[0]
        and q.shape[1] % k.shape[1] == 0
        and _lib.lib_has("sb200_fa_fwd")
    )


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: Optional[torch.Tensor],
                    cu_seqlens_k: Optional[torch.Tensor] = None, causal: bool = True,
                    scale: Optional[float] = None, window: Optional[int] = None,
                    dropout_p: float = 0.0,
                    doc_ranges: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
                    rng_state=None, head_offset: int = 0) -> torch.Tensor:
    """``doc_ranges = (doc_start[T], doc_end[T])`` (int32) may replace ``cu_seqlens_q`` for self-attention.

    ``dropout_p > 0`` drops attention probabilities; inside the kernel when ``rng_state`` (the topology's
    ``KernelDropoutState``) is given, where the mask is recomputed in the backward pass and costs no memory."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if (cu_seqlens_k is not None and cu_seqlens_q is not None and q.shape[0] == k.shape[0]
            and (cu_seqlens_k is cu_seqlens_q or cu_seqlens_q.numel() == cu_seqlens_k.numel() == 2)):
        cu_seqlens_k = None  # one document with as many keys as queries (filling a KV cache): plain self-attention
    d = q.shape[-1]
    if d < 128 and d != 64 and q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and cu_seqlens_k is None:
        # Head sizes between the two the kernel is built for: zero columns change neither the scores nor the
        # probabilities and give zero output columns, so the padded problem is the same attention.
        pad = (0, (64 if d < 64 else 128) - d)
        F = torch.nn.functional
        out = flash_attention(F.pad(q, pad), F.pad(k, pad), F.pad(v, pad), cu_seqlens_q, None, causal, scale, window,
                              dropout_p, doc_ranges, rng_state, head_offset)
        return out[..., :d]
    if (dropout_p == 0.0 or rng_state is not None) and kernel_supported(q, k, cu_seqlens_k):
        from .attention_kernel import dropout_args, flash_attention_kernel

        return flash_attention_kernel(q, k, v, cu_seqlens_q, causal, scale, window, doc_ranges,
                                      dropout_args(dropout_p, rng_state, head_offset))
    if cu_seqlens_k is not None and cu_seqlens_q is not None and dropout_p == 0.0 and q.is_cuda:
        from .attention_kernel import decode_supported, flash_decode

        if decode_supported(q, k, v):  # a few queries against many cached keys: streaming kernel, forward only
            return flash_decode(q, k, v, cu_seqlens_q, cu_seqlens_k, causal, scale, window)
    assert cu_seqlens_q is not None, "the dense attention path needs cumulative sequence lengths"
    if q.is_cuda and cu_seqlens_k is None and window is None:
        # head sizes the tcgen05 kernel does not cover: batched library attention over equal-length documents
        L = _uniform_docs(cu_seqlens_q, q.shape[0])
        if L is not None:
            n = q.shape[0] // L
            qb, kb, vb = (t.view(n, L, t.shape[1], t.shape[2]).transpose(1, 2) for t in (q, k, v))
            out = torch.nn.functional.scaled_dot_product_attention(
                qb, kb, vb, dropout_p=dropout_p, is_causal=causal, scale=scale, enable_gqa=q.shape[1] != k.shape[1]
            )
            return out.transpose(1, 2).reshape(q.shape)
    return attention_reference(q, k, v, cu_seqlens_q, cu_seqlens_k, causal, scale, window, dropout_p)
