"""Low-rank adapters that run in parallel to the attention projections.

``ParallelLoRa`` = ``B(A(x)) * alpha / rank`` with ``A`` drawn Kaiming-uniform and ``B`` zero, so
training starts at the base model.  Module layout and parameter names (``dense_in``, ``dense_out``)
follow the reference (src/scaling/core/nn/lora.py:12-166): for query/key/value both factors are
column-parallel (A gathered, B with parallel output); for the output projection ``dense`` A is
column-parallel with parallel output and B row-parallel.  ``get_delta_weights`` returns this rank's
slice of ``B @ A * scale`` for merging into the base weight.
"""

from __future__ import annotations

import math
from enum import Enum
from functools import partial
from typing import List, Optional, Union

import torch
import torch.distributed as dist
from pydantic import Field

from ...parallel.collectives import copy_to_tensor_model_parallel_region
from ...parallel.topology import Topology
from ..config import BaseConfig
from .linear import ColumnParallelLinear, RowParallelLinear


class LoRAModuleType(Enum):
    QUERY = "query"
    KEY = "key"
    VALUE = "value"
    DENSE = "dense"


class LoRaConfig(BaseConfig):
    name: str = Field(default="lora", description="name used in parameter and checkpoint file names")
    rank: int = Field(default=64, description="intrinsic rank of the adapter over all heads")
    parallel_modules: List[LoRAModuleType] = Field(
        default=[LoRAModuleType.DENSE, LoRAModuleType.KEY, LoRAModuleType.VALUE, LoRAModuleType.QUERY],
        description="projections that receive a parallel adapter",
    )
    dropout: float = Field(default=0.0, description="dropout probability between A and B")
    alpha: int = Field(default=1, description="scaling numerator (scale = alpha / rank)")
    bias: bool = Field(default=False, description="give the adapter linears a bias")
    kaiming_a: float = Field(default=math.sqrt(5), description="negative slope used for the Kaiming init of A")


def _gather_dim(t: torch.Tensor, dim: int, topology: Topology) -> torch.Tensor:
    parts = [torch.empty_like(t) for _ in range(topology.model_parallel_size)]
    dist.all_gather(parts, t.contiguous(), group=topology.model_parallel_group)
    return torch.cat(parts, dim=dim)


class ParallelLoRa(torch.nn.Module):
    def __init__(self, in_features: int, out_features: int, lora_module_type: LoRAModuleType, rank: int,
                 bias: bool = False, alpha: int = 1, dtype: torch.dtype = torch.float32, kaiming_a: float = 1.0e-5,
                 device: Optional[torch.device] = None, dropout: Optional[float] = None,
                 topology: Optional[Topology] = None) -> None:
        super().__init__()
        assert rank <= in_features, f"LoRa Rank: {rank} is greater or equal to the Input dimensionality: {in_features}"
        self.scaling = alpha / rank
        self.topology = topology
        self.model_parallel_size = 1 if topology is None else topology.config.model_parallel_size
        if self.model_parallel_size > 1:
            assert rank % self.model_parallel_size == 0, "LoRA rank must be divisible by the model parallel size"
            assert out_features % self.model_parallel_size == 0, "out_features must be divisible by the model parallel size"
        self.dropout = torch.nn.Dropout(dropout) if dropout else None
        self.lora_module_type = lora_module_type
        is_dense = lora_module_type == LoRAModuleType.DENSE
        common = dict(bias=bias, device=device, dtype=dtype, topology=topology)
        self.dense_in = ColumnParallelLinear(
            in_features=in_features, out_features=rank, parallel_output=is_dense,
            init_method=partial(torch.nn.init.kaiming_uniform_, a=kaiming_a), **common,
        )
        self.dense_out: Union[ColumnParallelLinear, RowParallelLinear]
        if is_dense:
            self.dense_out = RowParallelLinear(
                in_features=rank, out_features=out_features, init_method=torch.nn.init.zeros_, parallel_input=True,
                parallel_output=False, **common,
            )
        else:
            self.dense_out = ColumnParallelLinear(
                in_features=rank, out_features=out_features, init_method=torch.nn.init.zeros_, parallel_output=True,
                **common,
            )

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # Under sequence parallelism a column-parallel linear takes its input from the token gather, whose backward
        # pass sums the partial input gradients.  Two inputs here are replicated tensors instead (the full attention
        # output fed to the dense adapter, and the gathered low-rank activations fed to the second linear): their
        # gradient is summed explicitly.
        sp = (self.topology is not None and self.model_parallel_size > 1 and self.topology.config.sequence_parallel)
        is_dense = self.lora_module_type == LoRAModuleType.DENSE
        if sp and is_dense:
            x = copy_to_tensor_model_parallel_region(x, self.topology)
        x = self.dense_in(x)
        if self.dropout is not None:
            x = self.dropout(x)
        if sp and not is_dense:
            x = copy_to_tensor_model_parallel_region(x, self.topology)
        return self.dense_out(x) * self.scaling

    def get_delta_weights(self) -> torch.Tensor:
        """This rank's shard of the full-rank update ``(B @ A) * scale`` for the adapted base weight."""
        mp = self.model_parallel_size
        is_dense = self.lora_module_type == LoRAModuleType.DENSE
        a, b = self.dense_in.weight, self.dense_out.weight
        if mp > 1:
            assert self.topology is not None
            a = _gather_dim(a, -2, self.topology)
            b = _gather_dim(b, -1 if is_dense else -2, self.topology)
        delta = (b @ a) * self.scaling
        if mp == 1:
            return delta
        r = self.topology.model_parallel_rank  # type: ignore[union-attr]
        if is_dense:  # base weight is row parallel: slice input features
            w = delta.shape[1] // mp
            return delta[:, r * w:(r + 1) * w]
        w = delta.shape[0] // mp  # base weight is column parallel: slice output features
        return delta[r * w:(r + 1) * w]
