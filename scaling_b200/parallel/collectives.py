"""Autograd-aware collectives of the tensor-parallel / sequence-parallel region.

forward / backward pairs (reference: src/scaling/core/nn/linear/utils.py:195-361):
    copy_to_tensor_model_parallel_region     identity     / all-reduce
    all_reduce                               all-reduce   / identity
    all_concat                               all-gather of the last dim / local shard
    all_shard                                local shard of the last dim / all-gather
    all_reduce_scatter_to_sequence_parallel  reduce-scatter over tokens / all-gather
    gather_from_sequence_parallel_region     all-gather over tokens / reduce-scatter
Every function is the identity for a group of one.  The sequence-parallel shard is a contiguous
chunk of the flattened ``batch * sequence`` tokens (dimension 1 of ``[b, s, h]`` is divided by the
group size, memory is split rank-major), exactly like the reference.  With the gloo backend, which
has no reduce-scatter, an all-reduce followed by a local slice stands in.
"""

from __future__ import annotations

from typing import Any, Optional

import torch
import torch.distributed as dist

from .topology import Topology


def _size(topology: Optional[Topology]) -> int:
    return 1 if topology is None else topology.model_parallel_size


def _backend_is_gloo(group: Any) -> bool:
    return dist.get_backend(group) == "gloo"


# ------------------------------------------------------------------ raw (non-autograd) helpers
def all_reduce_raw(x: torch.Tensor, group: Any, op: Any = None) -> torch.Tensor:
    x = x.contiguous()
    dist.all_reduce(x, op=op or dist.ReduceOp.SUM, group=group)
    return x


def all_gather_last_dim_raw(x: torch.Tensor, topology: Topology) -> torch.Tensor:
    n = topology.model_parallel_size
    x = x.contiguous()
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x, group=topology.model_parallel_group)
    return torch.cat(parts, dim=-1)


def shard_last_dim_raw(x: torch.Tensor, topology: Topology) -> torch.Tensor:
    n, r = topology.model_parallel_size, topology.model_parallel_rank
    assert x.shape[-1] % n == 0, f"last dim {x.shape[-1]} not divisible by model parallel size {n}"
    w = x.shape[-1] // n
    return x[..., r * w:(r + 1) * w].contiguous()


def _sp_out_shape(shape: torch.Size, n: int, gather: bool) -> list[int]:
    out = list(shape)
    if gather:
        out[1] = out[1] * n
    else:
        assert out[1] % n == 0, f"sequence dim {out[1]} not divisible by model parallel size {n}"
        out[1] = out[1] // n
    return out


def reduce_scatter_tokens_raw(x: torch.Tensor, topology: Topology) -> torch.Tensor:
    n, r = topology.model_parallel_size, topology.model_parallel_rank
    group = topology.model_parallel_group
    x = x.contiguous()
    out_shape = _sp_out_shape(x.shape, n, gather=False)
    if _backend_is_gloo(group):
        dist.all_reduce(x, group=group)
        flat = x.view(-1)
        chunk = flat.numel() // n
        return flat[r * chunk:(r + 1) * chunk].clone().view(out_shape)
    out = torch.empty(out_shape, dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


def all_gather_tokens_raw(x: torch.Tensor, topology: Topology) -> torch.Tensor:
    n = topology.model_parallel_size
    group = topology.model_parallel_group
    x = x.contiguous()
    out = torch.empty(_sp_out_shape(x.shape, n, gather=True), dtype=x.dtype, device=x.device)
    if _backend_is_gloo(group):
        parts = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(parts, x, group=group)
        out.view(-1).copy_(torch.cat([p.view(-1) for p in parts]))
        return out
    dist.all_gather_into_tensor(out, x, group=group)
    return out


# ------------------------------------------------------------------ autograd functions
class _CopyToRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topology):  # type: ignore[override]
        ctx.topology = topology
        return x

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return all_reduce_raw(g, ctx.topology.model_parallel_group), None


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topology):  # type: ignore[override]
        return all_reduce_raw(x, topology.model_parallel_group)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return g, None


class _AllConcat(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topology):  # type: ignore[override]
        ctx.topology = topology
        return all_gather_last_dim_raw(x, topology)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return shard_last_dim_raw(g, ctx.topology), None


class _AllShard(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topology):  # type: ignore[override]
        ctx.topology = topology
        return shard_last_dim_raw(x, topology)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return all_gather_last_dim_raw(g, ctx.topology), None


class _ReduceScatterTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topology):  # type: ignore[override]
        ctx.topology = topology
        return reduce_scatter_tokens_raw(x, topology)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return all_gather_tokens_raw(g, ctx.topology), None


class _GatherTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topology, reduce_grad=True):  # type: ignore[override]
        ctx.topology = topology
        ctx.reduce_grad = reduce_grad
        return all_gather_tokens_raw(x, topology)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        if ctx.reduce_grad:
            return reduce_scatter_tokens_raw(g, ctx.topology), None, None
        t = ctx.topology
        n, r = t.model_parallel_size, t.model_parallel_rank
        flat = g.contiguous().view(-1)
        chunk = flat.numel() // n
        return flat[r * chunk:(r + 1) * chunk].clone().view(_sp_out_shape(g.shape, n, gather=False)), None, None


class _ShardTokens(torch.autograd.Function):
    """Keep this rank's contiguous chunk of the tokens of a replicated activation; backward gathers the chunks."""

    @staticmethod
    def forward(ctx, x, topology):  # type: ignore[override]
        ctx.topology = topology
        n, r = topology.model_parallel_size, topology.model_parallel_rank
        flat = x.contiguous().view(-1)
        chunk = flat.numel() // n
        return flat[r * chunk:(r + 1) * chunk].clone().view(_sp_out_shape(x.shape, n, gather=False))

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return all_gather_tokens_raw(g, ctx.topology), None


# ------------------------------------------------------------------ public API
def shard_to_sequence_parallel_region(x: torch.Tensor, topology: Optional[Topology]) -> torch.Tensor:
    """Replicated activation -> this rank's tokens (the layout a reduce-scatter over tokens leaves behind)."""
    return x if _size(topology) == 1 else _ShardTokens.apply(x, topology)


# The six functions below take ``(input_tensor, topology)``; ``all_concat`` / ``all_shard`` also the form
# ``(input_tensor, dim, topology)`` and ``gather_from_sequence_parallel_region`` the flag
# ``tensor_parallel_output_grad`` of src/scaling/core/nn/linear/utils.py:195-252, so layers written against those run.
def _dim_and_topology(args: tuple, kwargs: dict) -> tuple[int, Optional[Topology]]:
    dim = kwargs.pop("dim", None)
    topology = kwargs.pop("topology", None)
    rest = list(args)
    if rest and isinstance(rest[0], int) and not isinstance(rest[0], bool):
        dim = rest.pop(0)
    if rest:
        topology = rest.pop(0)
    assert not rest and not kwargs, f"unexpected arguments {rest} {kwargs}"
    return (-1 if dim is None else dim), topology


def _on_last_dim(fn, x: torch.Tensor, dim: int, topology: Topology) -> torch.Tensor:
    if dim in (-1, x.dim() - 1):
        return fn(x, topology)
    return fn(x.transpose(dim, -1), topology).transpose(dim, -1)


def copy_to_tensor_model_parallel_region(input_tensor: torch.Tensor, topology: Optional[Topology]) -> torch.Tensor:
    return input_tensor if _size(topology) == 1 else _CopyToRegion.apply(input_tensor, topology)


def all_reduce(input_tensor: torch.Tensor, topology: Optional[Topology]) -> torch.Tensor:
    return input_tensor if _size(topology) == 1 else _AllReduce.apply(input_tensor, topology)


def all_concat(input_tensor: torch.Tensor, *args, **kwargs) -> torch.Tensor:
    """Gather the shards of dimension ``dim`` (default: the last) from the tensor-parallel ranks; backward keeps
    this rank's shard of the gradient."""
    dim, topology = _dim_and_topology(args, kwargs)
    return input_tensor if _size(topology) == 1 else _on_last_dim(_AllConcat.apply, input_tensor, dim, topology)


def all_shard(input_tensor: torch.Tensor, *args, **kwargs) -> torch.Tensor:
    """Keep this rank's shard of dimension ``dim`` (default: the last); backward gathers the gradient shards."""
    dim, topology = _dim_and_topology(args, kwargs)
    return input_tensor if _size(topology) == 1 else _on_last_dim(_AllShard.apply, input_tensor, dim, topology)


def all_reduce_scatter_to_sequence_parallel(input_tensor: torch.Tensor, topology: Optional[Topology]) -> torch.Tensor:
    return input_tensor if _size(topology) == 1 else _ReduceScatterTokens.apply(input_tensor, topology)


def gather_from_sequence_parallel_region(input_tensor: torch.Tensor, topology: Optional[Topology],
                                         tensor_parallel_output_grad: bool = True) -> torch.Tensor:
    """Gather the token shards; the gradient is summed over the ranks and scattered back (the consumers are
    tensor-parallel and see different gradients) or, with ``tensor_parallel_output_grad=False``, only split (the
    consumers are replicated and every rank already holds the whole gradient)."""
    if _size(topology) == 1:
        return input_tensor
    return _GatherTokens.apply(input_tensor, topology, tensor_parallel_output_grad)


class SequenceShard:
    """This rank's tokens of an activation that is split over the tensor-parallel group (sequence parallelism), handed
    from a norm to the linears behind it without gathering first.  A consumer that can gather inside its GEMM takes
    ``shard``; every other consumer calls :meth:`gathered`, which runs the all-gather once and keeps the result for
    the consumers that follow."""

    def __init__(self, shard: torch.Tensor, topology: Topology):
        self.shard = shard
        self.topology = topology
        self._full: Optional[torch.Tensor] = None

    @property
    def shape(self) -> torch.Size:
        return torch.Size(_sp_out_shape(self.shard.shape, self.topology.model_parallel_size, gather=True))

    @property
    def device(self) -> torch.device:
        return self.shard.device

    @property
    def dtype(self) -> torch.dtype:
        return self.shard.dtype

    @property
    def is_cuda(self) -> bool:
        return self.shard.is_cuda

    def gathered(self) -> torch.Tensor:
        if self._full is None:
            self._full = gather_from_sequence_parallel_region(self.shard, self.topology)
        return self._full
