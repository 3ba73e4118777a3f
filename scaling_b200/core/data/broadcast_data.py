"""Hand a micro batch from tensor-parallel rank 0 to the rest of its tensor-parallel group.

Two broadcasts per dtype (src/scaling/core/data/broadcast_data.py:14-167): an int64 table with up to
``_MAX_DATA_DIM`` sizes per tensor (padded with -1), then one flat payload of all tensors (bool
travels as int8).  With a tensor-parallel group of one this degenerates to an asynchronous host to
device copy from pinned memory.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ...parallel.topology import Topology

_MAX_DATA_DIM = 8

TensorSizes = list[list[int]]
NumbersOfElements = list[int]


def _build_tensor_sizes(tensors: list[Optional[torch.Tensor]], model_parallel_rank: int) -> list[int]:
    """Flat size table: ``_MAX_DATA_DIM`` slots per tensor, unused slots -1; only rank 0 knows the sizes."""
    table = [-1] * (_MAX_DATA_DIM * len(tensors))
    if model_parallel_rank != 0:
        return table
    for i, t in enumerate(tensors):
        assert t is not None and t.dim() <= _MAX_DATA_DIM, "you should increase MAX_DATA_DIM"
        for j, s in enumerate(t.shape):
            assert s > 0, "cannot communicate tensor of size 0"
            table[i * _MAX_DATA_DIM + j] = int(s)
    return table


def _unpack_sizes(tensor_sizes: list[int]) -> tuple[TensorSizes, NumbersOfElements]:
    sizes: TensorSizes = []
    numels: NumbersOfElements = []
    for start in range(0, len(tensor_sizes), _MAX_DATA_DIM):
        shape = []
        n = 1
        for s in tensor_sizes[start:start + _MAX_DATA_DIM]:
            if s <= 0:
                break
            shape.append(s)
            n *= s
        sizes.append(shape)
        numels.append(n)
    return sizes, numels


def _src(topology: Topology) -> int:
    return dist.get_global_rank(topology.model_parallel_group, 0)


def sync_sizes(tensors: list[Optional[torch.Tensor]], topology: Topology) -> tuple[TensorSizes, NumbersOfElements]:
    table = torch.tensor(_build_tensor_sizes(tensors, topology.model_parallel_rank), dtype=torch.int64,
                         device=topology.device)
    dist.broadcast(table, _src(topology), group=topology.model_parallel_group)
    return _unpack_sizes(table.tolist())


def broadcast_data(tensors: list[Optional[torch.Tensor]], dtype: torch.dtype, topology: Topology) -> list[torch.Tensor]:
    dev = topology.device
    if topology.config.model_parallel_size == 1 or not topology.is_distributed_initialized:
        out = []
        for t in tensors:
            assert t is not None and t.dtype == dtype, (
                f"broadcast_data requires a list of tensors of the same dtype; expected {dtype} got {getattr(t, 'dtype', None)}"
            )
            out.append(t.to(dev, non_blocking=True))
        return out
    sizes, numels = sync_sizes(tensors, topology)
    wire_dtype = torch.int8 if dtype == torch.bool else dtype
    if topology.model_parallel_rank == 0:
        for t in tensors:
            assert t is not None and t.dtype == dtype, (
                f"broadcast_data requires a list of tensors of the same dtype; expected {dtype} got {getattr(t, 'dtype', None)}"
            )
        if len({t.device for t in tensors}) > 1:  # type: ignore[union-attr]
            tensors = [t.to(dev, non_blocking=True) for t in tensors]  # type: ignore[union-attr]
        flat = torch.cat([t.contiguous().view(-1) for t in tensors]).to(wire_dtype).to(dev, non_blocking=True)  # type: ignore[union-attr]
    else:
        flat = torch.empty(sum(numels), dtype=wire_dtype, device=dev)
    dist.broadcast(flat, _src(topology), group=topology.model_parallel_group)
    if dtype == torch.bool:
        flat = flat.to(torch.bool)
    out, offset = [], 0
    for shape, n in zip(sizes, numels):
        out.append(flat.narrow(0, offset, n).view(shape))
        offset += n
    return out
