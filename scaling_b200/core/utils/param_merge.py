"""Merge / split of tensor-parallel parameters for layout-independent checkpoints.

``merge_parameter`` returns the full tensor on the CPU (an all-gather of the shards inside the
tensor-parallel group, concatenated along the parameter's model-parallel dimension; replicated
parameters are simply cloned).  ``split_parameter`` cuts this rank's shard out of a full tensor.
Same results as src/scaling/core/utils/param_merge.py:7-97, which broadcasts shard by shard.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ...parallel.topology import Topology
from ..nn.parameter_meta import CoreParameterMeta


def merge_parameter(parameter: torch.Tensor, core_parameter_meta: CoreParameterMeta, topology: Topology) -> torch.Tensor:
    # clones keep torch.save from serialising the whole flat buffer a view may live in
    mp = topology.config.model_parallel_size
    if mp == 1 or not core_parameter_meta.is_model_parallel:
        return parameter.detach().clone().cpu()
    local = parameter.detach().contiguous()
    parts = [torch.empty_like(local) for _ in range(mp)]
    dist.all_gather(parts, local, group=topology.model_parallel_group)
    return torch.cat([p.cpu() for p in parts], dim=core_parameter_meta.model_parallel_dimension)


def split_parameter(parameter: torch.Tensor, core_parameter_meta: CoreParameterMeta, topology: Topology) -> torch.Tensor:
    mp = topology.config.model_parallel_size
    dim = core_parameter_meta.model_parallel_dimension
    assert dim is not None
    size = parameter.size(dim)
    assert size % mp == 0, (
        f"cannot slice tensor for parallelization, the loaded {core_parameter_meta.layer_class_name} "
        f"{core_parameter_meta.parameter_name} is of size ({size}) in dimension {dim}, "
        f"it needs to be divisible by the model parallel size ({mp})"
    )
    width = size // mp
    return parameter.narrow(dim, topology.model_parallel_rank * width, width).contiguous()
