"""Tensor-parallel linears whose collective runs inside the GEMM kernel.

``gemm_allreduce(x, w)`` computes ``sum over ranks of x_r @ w_r^T`` with one kernel launch per rank
(``sb200_gemm_allreduce``): partial output tiles go to symmetric memory, the owner of a tile adds the ranks' partial
tiles through the NVSwitch (``multimem.ld_reduce``, or peer loads in rank order) while later tiles are still being
multiplied, and stores the sum into every rank's output.  It replaces GEMM + NCCL all-reduce in the forward pass of
row-parallel linears (src/scaling/core/nn/linear/row_parallel_linear.py:169,286-289) and in the input gradient of
column-parallel linears (src/scaling/core/nn/linear/utils.py:44).
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_double, c_int, c_long, c_void_p
from typing import Any, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import functional as K
from ..ops._lib import check, lib
from .fused_zero import _SymmetricBuffer

_DECLARED = False
FLAG_STRIDE = 8192  # output tiles of 128 rows a single fused GEMM may have
FUSED_TP_MAX_ELEMENTS = 2 * 1024 * 1024  # largest output (elements) routed to the fused kernel by default


def _declare() -> None:
    global _DECLARED
    if not _DECLARED:
        _lib.declare("sb200_gemm_allreduce",
                     [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_long, c_long, c_long, c_int, c_int,
                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                      c_double, c_int, c_void_p, c_void_p])
        _DECLARED = True


class FusedTPWorkspace:
    """Symmetric buffers of one tensor-parallel group: partial products, reduced output, flags."""

    def __init__(self, group: dist.ProcessGroup, device: torch.device, max_elements: int, use_multicast: bool = True):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.max_elements = int(max_elements)
        self.partial = _SymmetricBuffer(self.max_elements, torch.bfloat16, device, group)
        self.out = _SymmetricBuffer(self.max_elements, torch.bfloat16, device, group)
        self.flags = _SymmetricBuffer((self.world + 1) * FLAG_STRIDE, torch.int32, device, group)
        self.flags.tensor.zero_()
        self.local = torch.zeros(2, dtype=torch.int32, device=device)  # [epoch, finished CTAs]
        self.use_multicast = (use_multicast and self.partial.multicast_ptr is not None
                              and self.out.multicast_ptr is not None)
        self.timeout_s = float(os.environ.get("SB200_P2P_TIMEOUT_S", "10"))
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def gemm_allreduce(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                       b_mn: bool = False) -> torch.Tensor:
        """``x [M, K] @ op(w)`` summed over the group; ``w`` is ``[N, K]`` (``b_mn=False``) or ``[K, N]``."""
        _declare()
        M, Kd = x.shape
        N = w.shape[1] if b_mn else w.shape[0]
        assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
        assert M * N <= self.max_elements, f"fused workspace holds {self.max_elements} elements, need {M * N}"
        mc = self.use_multicast
        check(lib().sb200_gemm_allreduce(
            x.data_ptr(), w.data_ptr(), _lib.ptr(bias), M, N, Kd, x.stride(0), w.stride(0), N, int(b_mn),
            _lib.dt(x.dtype), self.partial.c_ptrs, self.out.c_ptrs, self.flags.c_ptrs,
            self.partial.multicast_ptr if mc else None, self.out.multicast_ptr if mc else None, FLAG_STRIDE,
            self.local.data_ptr(), self.local.data_ptr() + 4, self.rank, self.world, self.timeout_s, _lib.sm_count(),
            K.status_word().data_ptr(), _lib.stream()), "sb200_gemm_allreduce")
        return self.out.tensor[:M * N].view(M, N).clone()


_WORKSPACES: dict[Any, Optional[FusedTPWorkspace]] = {}


def workspace_for(topology: Any, elements: int) -> Optional[FusedTPWorkspace]:
    """The fused workspace of the topology's tensor-parallel group (created on first use by all ranks of the group
    together), or None where the fused path does not apply."""
    if os.environ.get("SB200_FUSED_TP", "1") == "0":
        return None
    if topology is None or topology.config.model_parallel_size < 2 or topology.device.type != "cuda":
        return None
    if topology.config.model_parallel_size > 8 or not _lib.lib_has("sb200_gemm_allreduce"):
        return None
    key = id(topology)
    ws = _WORKSPACES.get(key)
    if key not in _WORKSPACES or (ws is not None and ws.max_elements < elements):
        try:
            size = max(elements, int(os.environ.get("SB200_FUSED_TP_ELEMENTS", str(64 * 1024 * 1024))))
            ws = FusedTPWorkspace(topology.model_parallel_group, topology.device, size,
                                  os.environ.get("SB200_P2P_MULTICAST", "1") != "0")
        except Exception as e:  # noqa: BLE001 - no peer access / symmetric memory on this machine
            from ..core.logging import logger

            logger.warning(f"fused tensor-parallel GEMMs unavailable ({type(e).__name__}: {e}); using NCCL")
            ws = None
        _WORKSPACES[key] = ws
    return ws


class _RowParallelLinearFn(torch.autograd.Function):
    """``all_reduce(x @ w^T) (+ bias once)`` with the reduction inside the GEMM; backward has no communication."""

    @staticmethod
    def forward(ctx, x, w, bias, ws: FusedTPWorkspace):  # type: ignore[override]
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = ws.gemm_allreduce(x2, w, bias if ws.rank == 0 else None)
        ctx.save_for_backward(x2, w)
        ctx.weight, ctx.bias = w, bias
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = K.gemm(dy2, w, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            main = K.fused_grad_target(ctx.weight)
            if main is not None and main.dtype in (torch.float32, dy2.dtype):
                K.gemm(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=True)
            else:
                dw = K.gemm(dy2, x2, a_mn=True, b_mn=True)
        if ctx.bias is not None and ctx.needs_input_grad[2]:
            main = K.fused_grad_target(ctx.bias)
            if main is not None and main.dtype == dy2.dtype:
                K.column_sum(dy2, out=main, accumulate=True)
            else:
                db = K.column_sum(dy2)
        return dx, dw, db, None


def row_parallel_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], topology: Any) -> Optional[torch.Tensor]:
    """Fused row-parallel linear, or None when the caller has to take the GEMM + collective path."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous()):
        return None
    M = x.numel() // x.shape[-1]
    N, Kd = w.shape
    if N % 8 or Kd % 8 or (bias is not None and bias.dtype != torch.bfloat16):
        return None
    if (M + 127) // 128 * ((N + 127) // 128) > FLAG_STRIDE:
        return None
    # Measured on 2 x B200: the fused kernel wins for outputs up to a few MB (27-41 us against 42-48 us for GEMM + NCCL
    # at 128 x 64 ... 256 x 256) and loses for the 25 MB outputs of full training batches (120 us against 90-110 us),
    # where its reduction phase is still bound by NVLink round-trip latency.  SB200_FUSED_TP=always lifts the limit.
    mode = os.environ.get("SB200_FUSED_TP", "1")
    if mode != "always" and M * N > FUSED_TP_MAX_ELEMENTS:
        return None
    ws = workspace_for(topology, M * N)
    if ws is None or M * N > ws.max_elements:
        return None
    return _RowParallelLinearFn.apply(x, w, bias, ws)


class _ColumnParallelLinearFn(torch.autograd.Function):
    """Column-parallel ``act(x @ w^T + b)``: no communication forward; the input gradient ``dy @ w`` is summed over the
    tensor-parallel ranks inside the GEMM kernel (the backward of the identity that feeds replicated activations into
    a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, w, bias, act: str, ws: FusedTPWorkspace):  # type: ignore[override]
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        pre = torch.empty((x2.shape[0], w.shape[0]), dtype=x.dtype, device=x.device) if act == "gelu" else None
        y = K.gemm(x2, w, bias=bias, act=act, pre_act_out=pre)
        ctx.save_for_backward(x2, w, pre)
        ctx.weight, ctx.bias, ctx.act, ctx.ws, ctx.x_shape = w, bias, act, ws, x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x2, w, pre = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.act == "gelu":
            dy2 = K.gelu_backward(dy2, pre)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = ctx.ws.gemm_allreduce(dy2, w, None, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            main = K.fused_grad_target(ctx.weight)
            if main is not None and main.dtype in (torch.float32, dy2.dtype):
                K.gemm(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=True)
            else:
                dw = K.gemm(dy2, x2, a_mn=True, b_mn=True)
        if ctx.bias is not None and ctx.needs_input_grad[2]:
            main = K.fused_grad_target(ctx.bias)
            if main is not None and main.dtype == dy2.dtype:
                K.column_sum(dy2, out=main, accumulate=True)
            else:
                db = K.column_sum(dy2)
        return dx, dw, db, None, None


def column_parallel_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], act: str,
                           topology: Any) -> Optional[torch.Tensor]:
    """Column-parallel linear whose input-gradient all-reduce is fused into the dgrad GEMM, or None when the caller
    has to take the unfused path (``x`` must be the replicated activation itself, not the output of the identity
    whose backward reduces)."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous()):
        return None
    if not x.requires_grad or act not in ("none", "gelu"):
        return None
    M = x.numel() // x.shape[-1]
    N, Kd = w.shape
    if N % 8 or Kd % 8 or (bias is not None and bias.dtype != torch.bfloat16):
        return None
    mode = os.environ.get("SB200_FUSED_TP", "1")
    if mode != "always" and M * Kd > FUSED_TP_MAX_ELEMENTS:
        return None
    if (M + 127) // 128 * ((Kd + 127) // 128) > FLAG_STRIDE:
        return None
    ws = workspace_for(topology, M * Kd)
    if ws is None or M * Kd > ws.max_elements:
        return None
    return _ColumnParallelLinearFn.apply(x, w, bias, act, ws)
