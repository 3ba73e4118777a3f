"""Tensor-parallel linears whose collective runs inside the GEMM kernel (``sb200_gemm_tp``, one launch per rank).

* ``gemm_allreduce(x, w)``: ``sum over ranks of x_r @ w_r^T``.  Partial output tiles go to symmetric memory, the
  owner of a tile adds the ranks' partial tiles through the NVSwitch (``multimem.ld_reduce``, or peer loads in rank
  order) while later tiles are still being multiplied, and stores the sum into every rank's output.  Forward of
  row-parallel linears (src/scaling/core/nn/linear/row_parallel_linear.py:169,286-289) and input gradient of
  column-parallel linears (src/scaling/core/nn/linear/utils.py:44).
* ``gemm_reduce_scatter(x, w)``: the same sum, of which a rank keeps its block of rows (tokens): the row-parallel
  linear under sequence parallelism (src/scaling/core/nn/linear/utils.py:156-192) and the input gradient of the
  column-parallel one.
* ``allgather_gemm(shard, w)``: ``[shard_0; shard_1; ...] @ w^T``.  Extra warps push this rank's rows into every
  rank's copy of the operand (``multimem.st`` or peer stores) and the tile loads of a row block wait for its flag:
  the column-parallel linear on sequence-sharded input, and the input gradient of the row-parallel one.
"""

from __future__ import annotations

import os
from ctypes import c_double, c_int, c_long, c_void_p
from typing import Any, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import functional as K
from ..ops._lib import check, lib
from .fused_zero import _SymmetricBuffer, device_wait_limit_s

_DECLARED = False
FLAG_STRIDE = 8192  # output tiles of 128 rows a single fused GEMM may have
FUSED_TP_MAX_ELEMENTS = 2 * 1024 * 1024  # largest output (elements) routed to the fused kernel by default


MODE_ALLREDUCE, MODE_REDUCE_SCATTER, MODE_ALLGATHER = 0, 1, 2
_VERIFY = os.environ.get("SB200_FUSED_TP_VERIFY", "0") == "1"
_ACT = {"none": 0, "gelu": 1}


def _declare() -> None:
    global _DECLARED
    if not _DECLARED:
        _lib.declare("sb200_gemm_tp",
                     [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_long, c_long, c_long,
                      c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                      c_void_p, c_int, c_int, c_long, c_int, c_int, c_double, c_int, c_void_p, c_void_p])
        _DECLARED = True


class FusedTPWorkspace:
    """Symmetric buffers of one tensor-parallel group: partial products / gathered operand, reduced output, flags."""

    def __init__(self, group: dist.ProcessGroup, device: torch.device, max_elements: int, use_multicast: bool = True,
                 reserved_sms: int = 0):
        self.group = group
        # SMs the fused kernels leave free: their CTAs wait for CTAs of other GPUs, so all of them must be resident
        # at once even while kernels of other streams (point-to-point copies between pipeline stages) hold SMs
        self.reserved_sms = int(reserved_sms)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.max_elements = int(max_elements)
        # two buffers that consecutive launches use in turn (see _launch)
        self.partial = _SymmetricBuffer(2 * self.max_elements, torch.bfloat16, device, group)
        self.out = _SymmetricBuffer(self.max_elements, torch.bfloat16, device, group)
        self.flags = _SymmetricBuffer((self.world + 2) * FLAG_STRIDE, torch.int32, device, group)
        self.flags.tensor.zero_()
        self.local = torch.zeros(2, dtype=torch.int32, device=device)  # [epoch, finished CTAs]
        self.use_multicast = (use_multicast and self.partial.multicast_ptr is not None
                              and self.out.multicast_ptr is not None)
        self.timeout_s = device_wait_limit_s()
        self.launches = 0
        self._count = 0        # launches since the alternation of the two buffers was last started
        self._last_half = 0
        self._gathered_key: Any = None
        self._regathered: Any = None
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    # ------------------------------------------------------------------ the kernel
    def _launch(self, mode: int, a: torch.Tensor, w: torch.Tensor, c: Optional[torch.Tensor],
                c_pre: Optional[torch.Tensor], bias: Optional[torch.Tensor], M: int, N: int, Kd: int, b_mn: bool,
                act: str) -> None:
        _declare()
        assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.stride(1) == 1 and w.stride(1) == 1
        need = M * Kd if mode == MODE_ALLGATHER else M * N
        assert need <= self.max_elements, f"fused workspace holds {self.max_elements} elements, need {need}"
        mc = self.use_multicast
        self.launches += 1
        # Partial products / the gathered operand go to the two halves of `partial` in turn, which is what lets the
        # reduce-scatter and all-gather forms run without a handshake at their start and end.  The first launch after
        # restart_alternation() (start of a step) begins at half 0 and makes all ranks wait for each other once, so
        # that a captured step can be replayed whatever its number of launches.
        half, sync_entry = self._count & 1, int(self._count == 0)
        self._count += 1
        self._last_half = half
        check(lib().sb200_gemm_tp(
            a.data_ptr(), w.data_ptr(), _lib.ptr(c), _lib.ptr(c_pre), _lib.ptr(bias), M, N, Kd, a.stride(0),
            w.stride(0), N, int(b_mn), _ACT[act], _lib.dt(a.dtype), mode, self.partial.c_ptrs, self.out.c_ptrs,
            self.flags.c_ptrs, self.partial.multicast_ptr if mc else None, self.out.multicast_ptr if mc else None,
            FLAG_STRIDE, self.local.data_ptr(), self.local.data_ptr() + 4, self.rank, self.world, self.max_elements,
            half, sync_entry, self.timeout_s, max(2, _lib.sm_count() - self.reserved_sms) // 2 * 2,
            K.status_word().data_ptr(), _lib.stream()), "sb200_gemm_tp")

    def restart_alternation(self) -> None:
        """The next launch starts a new count of the buffer alternation (all ranks call this at the same point)."""
        self._count = 0

    def _verify(self, what: str, got: torch.Tensor, ref: torch.Tensor, shape: tuple) -> None:
        """SB200_FUSED_TP_VERIFY=1: every fused launch is compared with GEMM + NCCL (debugging aid; slow)."""
        torch.cuda.synchronize()
        K.check_status()
        err = (got.float() - ref.float()).norm() / ref.float().norm().clamp_min(1e-20)
        bad = torch.tensor([float(not torch.isfinite(err) or err > 1e-2)], device=got.device)
        dist.all_reduce(bad, group=self.group)
        if bad.item() > 0:
            raise RuntimeError(f"fused tensor-parallel GEMM ({what}, M/N/K/b_mn={shape}, launch {self.launches}) "
                               f"differs from GEMM + NCCL on rank {self.rank}: relative error {err.item():.3e}")

    def gemm_allreduce(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                       b_mn: bool = False) -> torch.Tensor:
        """``x [M, K] @ op(w)`` summed over the group; ``w`` is ``[N, K]`` (``b_mn=False``) or ``[K, N]``."""
        M, Kd = x.shape
        N = w.shape[1] if b_mn else w.shape[0]
        self._launch(MODE_ALLREDUCE, x, w, None, None, bias, M, N, Kd, b_mn, "none")
        out = self.out.tensor[:M * N].view(M, N).clone()
        if _VERIFY:
            ref = K.gemm(x, w, b_mn=b_mn, bias=bias)
            dist.all_reduce(ref, group=self.group)
            self._verify("all-reduce", out, ref, (M, N, Kd, b_mn))
        return out

    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                            b_mn: bool = False) -> torch.Tensor:
        """Rows ``[rank * M / W, (rank + 1) * M / W)`` of the summed product; ``M`` is a multiple of ``128 * W``."""
        M, Kd = x.shape
        N = w.shape[1] if b_mn else w.shape[0]
        out = torch.empty((M // self.world, N), dtype=x.dtype, device=x.device)
        self._launch(MODE_REDUCE_SCATTER, x, w, out, None, bias, M, N, Kd, b_mn, "none")
        if _VERIFY:
            ref = K.gemm(x, w, b_mn=b_mn, bias=bias)
            dist.all_reduce(ref, group=self.group)
            rows = M // self.world
            self._verify("reduce-scatter", out, ref[self.rank * rows:(self.rank + 1) * rows], (M, N, Kd, b_mn))
        return out

    def allgather_gemm(self, shard: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                       act: str = "none", pre_act_out: Optional[torch.Tensor] = None,
                       b_mn: bool = False) -> torch.Tensor:
        """``act(concat over ranks of shard_r [M / W, K] @ op(w) + bias)``; the gathered operand stays available
        through :meth:`gathered` until the next launch on this workspace."""
        Ms, Kd = shard.shape
        M = Ms * self.world
        N = w.shape[1] if b_mn else w.shape[0]
        out = torch.empty((M, N), dtype=shard.dtype, device=shard.device)
        self._launch(MODE_ALLGATHER, shard, w, out, pre_act_out, bias, M, N, Kd, b_mn, act)
        self._gathered_key = (shard.data_ptr(), shard._version, Ms, Kd, self.launches)
        if _VERIFY:
            full = torch.empty((M, Kd), dtype=shard.dtype, device=shard.device)
            dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
            self._verify("all-gather operand", self.gathered(M, Kd), full, (M, N, Kd, b_mn))
            self._verify("all-gather", out, K.gemm(full, w, b_mn=b_mn, bias=bias, act=act), (M, N, Kd, b_mn))
        return out

    def gathered(self, M: int, Kd: int) -> torch.Tensor:
        """The operand gathered by the last :meth:`allgather_gemm` (a view of the workspace)."""
        base = self._last_half * self.max_elements
        return self.partial.tensor[base:base + M * Kd].view(M, Kd)

    def cached_gather(self, shard: torch.Tensor) -> Optional[torch.Tensor]:
        """The gathered rows of ``shard`` if the previous launch on this workspace gathered exactly this tensor
        (linears that share their input, like query / key / value): peers write into the buffer again only after
        this rank has entered its next fused launch, which the stream orders after the readers of the view."""
        Ms, Kd = shard.shape
        if self._gathered_key == (shard.data_ptr(), shard._version, Ms, Kd, self.launches):
            return self.gathered(Ms * self.world, Kd)
        return None

    def regather(self, shard: torch.Tensor) -> torch.Tensor:
        """All ranks' rows of ``shard`` for a weight gradient; one gathered copy is kept for linears that share
        the same input."""
        key = (shard.data_ptr(), shard._version, tuple(shard.shape))
        if self._regathered is not None and self._regathered[0] == key:
            return self._regathered[1]
        full = torch.empty((shard.shape[0] * self.world, shard.shape[1]), dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(full, shard, group=self.group)
        # the entry holds the shard itself: its address cannot be handed to another tensor while the copy is cached
        self._regathered = (key, full, shard)
        return full

    def drop_regathered(self) -> None:
        self._regathered = None


_WORKSPACES: dict[Any, Optional[FusedTPWorkspace]] = {}


def begin_step() -> None:
    """Start of a training or evaluation step (called by the engine on every rank): the fused workspaces start their
    buffer alternation anew, so every step issues the same launches whether it runs eagerly or as a replayed graph."""
    for ws in _WORKSPACES.values():
        if ws is not None:
            ws.restart_alternation()


def workspace_for(topology: Any, elements: int) -> Optional[FusedTPWorkspace]:
    """The fused workspace of the topology's tensor-parallel group (created on first use by all ranks of the group
    together), or None where the fused path does not apply."""
    if os.environ.get("SB200_FUSED_TP", "1") == "0":
        return None
    if topology is None or topology.config.model_parallel_size < 2 or topology.device.type != "cuda":
        return None
    if topology.config.model_parallel_size > 8 or not _lib.lib_has("sb200_gemm_tp"):
        return None
    key = id(topology)
    ws = _WORKSPACES.get(key)
    if key not in _WORKSPACES or (ws is not None and ws.max_elements < elements):
        try:
            size = max(elements, int(os.environ.get("SB200_FUSED_TP_ELEMENTS", str(64 * 1024 * 1024))))
            # With pipeline stages, send / receive kernels of other streams share the SMs with the fused kernels,
            # whose CTAs wait for their peers' CTAs: the grid leaves as many SMs free as those copies can occupy
            # (Topology.reserved_sms), so that no wait depends on a CTA that cannot become resident.
            ws = FusedTPWorkspace(topology.model_parallel_group, topology.device, size,
                                  os.environ.get("SB200_P2P_MULTICAST", "1") != "0",
                                  reserved_sms=getattr(topology, "reserved_sms", 0))
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


# ---------------------------------------------------------------------------------------------- sequence parallel
def _wgrad(ctx_weight, dy2: torch.Tensor, x2: torch.Tensor) -> Optional[torch.Tensor]:
    main = K.fused_grad_target(ctx_weight)
    if main is not None and main.dtype in (torch.float32, dy2.dtype):
        K.gemm(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=True)
        return None
    return K.gemm(dy2, x2, a_mn=True, b_mn=True)


def _bgrad(ctx_bias, dy2: torch.Tensor) -> Optional[torch.Tensor]:
    main = K.fused_grad_target(ctx_bias)
    if main is not None and main.dtype == dy2.dtype:
        K.column_sum(dy2, out=main, accumulate=True)
        return None
    return K.column_sum(dy2)


class _RowParallelSPFn(torch.autograd.Function):
    """``reduce_scatter over tokens of (x @ w^T) (+ bias once)`` in one kernel; the backward pass gathers the output
    gradient inside the input-gradient GEMM and reuses the gathered copy for the weight gradient."""

    @staticmethod
    def forward(ctx, x, w, bias, ws: FusedTPWorkspace, out_shape):  # type: ignore[override]
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = ws.gemm_reduce_scatter(x2, w, bias if ws.rank == 0 else None)
        ctx.save_for_backward(x2, w)
        ctx.weight, ctx.bias, ctx.ws, ctx.x_shape = w, bias, ws, x.shape
        return y.view(out_shape)

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x2, w = ctx.saved_tensors
        ws = ctx.ws
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        M = dy2.shape[0] * ws.world
        dx = ws.allgather_gemm(dy2, w, b_mn=True).view(ctx.x_shape)  # [M, K_local]
        dy_full = ws.gathered(M, dy2.shape[1])
        dw = _wgrad(ctx.weight, dy_full, x2) if ctx.needs_input_grad[1] else None
        db = None
        if ctx.bias is not None and ctx.needs_input_grad[2] and ws.rank == 0:  # the bias entered on rank 0 only
            db = _bgrad(ctx.bias, dy_full)
        return dx, dw, db, None, None


class _ColumnParallelSPFn(torch.autograd.Function):
    """``act([x_0; x_1; ...] @ w^T + b)`` on sequence-sharded input with the all-gather inside the GEMM; the input
    gradient leaves through a GEMM with in-kernel reduce-scatter."""

    @staticmethod
    def forward(ctx, shard, w, bias, act: str, ws: FusedTPWorkspace, out_shape):  # type: ignore[override]
        s2 = shard.reshape(-1, shard.shape[-1])
        if not s2.is_contiguous():
            s2 = s2.contiguous()
        M = s2.shape[0] * ws.world
        pre = torch.empty((M, w.shape[0]), dtype=s2.dtype, device=s2.device) if act == "gelu" else None
        full = ws.cached_gather(s2)
        if full is not None:
            if _VERIFY:
                ref = torch.empty_like(full)
                dist.all_gather_into_tensor(ref, s2, group=ws.group)
                ws._verify("reused gathered operand", full, ref, (M, w.shape[0], s2.shape[1], False))
            y = K.gemm(full, w, bias=bias, act=act, pre_act_out=pre)
        else:
            y = ws.allgather_gemm(s2, w, bias, act, pre)
        ctx.save_for_backward(s2, w, pre)
        ctx.weight, ctx.bias, ctx.act, ctx.ws, ctx.shard_shape = w, bias, act, ws, shard.shape
        return y.view(*out_shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        s2, w, pre = ctx.saved_tensors
        ws = ctx.ws
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.act == "gelu":
            dy2 = K.gelu_backward(dy2, pre)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = ws.gemm_reduce_scatter(dy2, w, None, b_mn=True).view(ctx.shard_shape)
        if ctx.needs_input_grad[1]:
            dw = _wgrad(ctx.weight, dy2, ws.regather(s2))
        if ctx.bias is not None and ctx.needs_input_grad[2]:
            db = _bgrad(ctx.bias, dy2)
        return dx, dw, db, None, None, None


def _sp_eligible(rows: int, n: int, k: int, operand_elements: int, tensors, topology: Any) -> Optional[FusedTPWorkspace]:
    for t in tensors:
        if t is not None and not (t.is_cuda and t.dtype == torch.bfloat16):
            return None
    W = topology.config.model_parallel_size
    if rows % (128 * W) or n % 8 or k % 8:
        return None
    if (rows // 128) * ((n + 127) // 128) > FLAG_STRIDE:
        return None
    ws = workspace_for(topology, operand_elements)
    if ws is None or operand_elements > ws.max_elements:
        return None
    return ws


def row_parallel_linear_sp(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], topology: Any,
                           out_shape: list[int]) -> Optional[torch.Tensor]:
    """Row-parallel linear followed by the reduce-scatter over tokens, in one kernel; None where that cannot run."""
    M = x.numel() // x.shape[-1]
    N, Kd = w.shape
    if not w.is_contiguous():
        return None
    ws = _sp_eligible(M, N, Kd, max(M * N, M * Kd), (x, w, bias), topology)
    if ws is None:
        return None
    return _RowParallelSPFn.apply(x, w, bias, ws, out_shape)


def column_parallel_linear_sp(shard: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], act: str,
                              topology: Any, full_shape: list[int]) -> Optional[torch.Tensor]:
    """Column-parallel linear on this rank's tokens of a sequence-sharded input, the all-gather inside the kernel."""
    if act not in _ACT or not w.is_contiguous():
        return None
    W = topology.config.model_parallel_size
    M = shard.numel() // shard.shape[-1] * W
    N, Kd = w.shape
    ws = _sp_eligible(M, N, Kd, M * Kd, (shard, w, bias), topology)
    if ws is None:
        return None
    return _ColumnParallelSPFn.apply(shard, w, bias, act, ws, full_shape)
