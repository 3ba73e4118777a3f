"""ZeRO-1 gradient reduce-scatter and parameter all-gather as kernels over NVLink peer memory.

The flat gradient and parameter buffers of every parameter group move into symmetric memory (same allocation on
every rank of the data-parallel group, mapped into each other's address space).  The optimizer step then runs

    barrier -> reduce-scatter kernel (reads every peer's gradients, sums in rank order: deterministic)
            -> norm / AdamW on the owned range
            -> all-gather kernel (stores the new parameters into every peer's buffer, or once through the
               NVLink multicast mapping where the allocation has one)
            -> barrier

all of which are ordinary kernel launches on the compute stream: they are captured with the rest of the training
step in a CUDA graph, and no library collective is called for the data-parallel exchange.

Reference behaviour covered: src/scaling/core/optimizer/allreduce.py:16-38 (gradient reduction over the
data-parallel group) and src/scaling/core/optimizer/parameter_group.py:439-477 (parameter all-gather of the ZeRO
partitions).
"""

from __future__ import annotations

import ctypes
import os
from typing import Any, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import check, lib
from ..ops.functional import status_word


MAX_DEVICE_WAIT_S = 60.0


def device_wait_limit_s() -> float:
    """Limit of a device-side wait on a peer in seconds (``SB200_P2P_TIMEOUT_S``, default 10).  The kernels accept at
    most 60 s (a longer spin would look like a hung GPU to everything else on the machine); larger or non-positive
    settings are clamped, with a warning."""
    raw = os.environ.get("SB200_P2P_TIMEOUT_S", "10")
    try:
        value = float(raw)
    except ValueError:
        value = -1.0
    if 0.0 < value <= MAX_DEVICE_WAIT_S:
        return value
    clamped = MAX_DEVICE_WAIT_S if value > MAX_DEVICE_WAIT_S else 10.0
    from ..core.logging import logger

    logger.warning(f"SB200_P2P_TIMEOUT_S={raw!r} is outside (0, {MAX_DEVICE_WAIT_S:g}] seconds; using {clamped:g}")
    return clamped


def _ptr_array(ptrs: list[int]) -> Any:
    arr = (ctypes.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


class _SymmetricBuffer:
    """A tensor in symmetric memory plus the addresses under which the group's ranks (and the multicast object) see it."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group: dist.ProcessGroup):
        import torch.distributed._symmetric_memory as symm_mem

        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.rank = int(self.handle.rank)
        self.world = int(self.handle.world_size)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        assert self.peer_ptrs[self.rank] == self.tensor.data_ptr()
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.multicast_ptr: Optional[int] = mc if mc != 0 else None
        self.c_ptrs = _ptr_array(self.peer_ptrs)


class FusedZero:
    """Data-parallel exchange of the ZeRO step through the kernels of ``csrc/p2p.cu``."""

    def __init__(self, optimizer: Any, group: dist.ProcessGroup, use_multicast: bool):
        t = optimizer.topology
        dev = t.device
        self.group = group
        self.world = t.config.data_parallel_size
        self.rank = t.data_parallel_rank
        assert self.world <= lib().sb200_p2p_max_ranks()
        self.params: list[_SymmetricBuffer] = []
        self.grads: list[_SymmetricBuffer] = []
        for g in optimizer.parameter_groups:
            assert g.zero, "the fused path covers ZeRO parameter groups"
            fp = _SymmetricBuffer(g.flat_param.numel(), g.flat_param.dtype, dev, group)
            fg = _SymmetricBuffer(g.flat_grad.numel(), g.flat_grad.dtype, dev, group)
            assert fp.rank == self.rank and fp.world == self.world
            g.rehome(fp.tensor, fg.tensor)
            self.params.append(fp)
            self.grads.append(fg)
        self.flags = _SymmetricBuffer(64, torch.int32, dev, group)
        self.flags.tensor.zero_()
        self.round = torch.zeros(1, dtype=torch.int32, device=dev)
        self.use_multicast = use_multicast and all(b.multicast_ptr is not None for b in self.params)
        self.timeout_s = device_wait_limit_s()
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)  # every rank's flag words are zero before the first in-kernel barrier

    @classmethod
    def create(cls, optimizer: Any) -> Optional["FusedZero"]:
        t = optimizer.topology
        if not (_lib.available() and _lib.lib_has("sb200_p2p_barrier")):
            return None
        if t.config.data_parallel_size < 2 or t.device.type != "cuda":
            return None
        if os.environ.get("SB200_FUSED_ZERO", "1") == "0":
            return None
        use_mc = os.environ.get("SB200_P2P_MULTICAST", "1") != "0"
        return cls(optimizer, t.data_parallel_group, use_mc)

    # ------------------------------------------------------------------ pieces of the step
    def barrier(self) -> None:
        check(lib().sb200_p2p_barrier(self.flags.c_ptrs, self.round.data_ptr(), self.rank, self.world,
                                      status_word().data_ptr(), self.timeout_s, _lib.stream()), "sb200_p2p_barrier")

    def reduce_scatter(self, optimizer: Any) -> list[torch.Tensor]:
        """Owned range of every group's gradient, summed over the data-parallel ranks (into ``reduced_grad``)."""
        t = optimizer.topology
        for g in optimizer.parameter_groups:  # tensor-parallel partial gradients first, as on the library path
            a, b = g.segment_ends[1], g.segment_ends[2]
            if b > a and t.config.model_parallel_size > 1:
                dist.all_reduce(g.flat_grad[a:b], group=t.model_parallel_group)
        self.barrier()  # every rank's backward pass is complete
        out = []
        for g, buf in zip(optimizer.parameter_groups, self.grads):
            lo, hi = g.owned_range
            assert g.reduced_grad is not None
            check(lib().sb200_p2p_reduce_scatter(buf.c_ptrs, g.reduced_grad.data_ptr(), lo, hi - lo, self.world,
                                                 _lib.dt(g.flat_grad.dtype), _lib.sm_count(), _lib.stream()),
                  "sb200_p2p_reduce_scatter")
            out.append(g.reduced_grad)
        return out

    def all_gather(self, optimizer: Any) -> None:
        """Publish the updated owned parameter range of every group to all ranks."""
        for g, buf in zip(optimizer.parameter_groups, self.params):
            lo, hi = g.owned_range
            es = g.flat_param.element_size()
            mc = buf.multicast_ptr if self.use_multicast else None
            check(lib().sb200_p2p_all_gather(buf.c_ptrs, buf.tensor.data_ptr(), mc, lo * es, (hi - lo) * es, self.rank,
                                             self.world, _lib.sm_count(), _lib.stream()), "sb200_p2p_all_gather")
        # all stores have landed everywhere and every rank is done reading gradients: parameters may be read and
        # gradients cleared
        self.barrier()
