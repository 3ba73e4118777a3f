"""Helpers of the parallel linear layers under the module path of src/scaling/core/nn/linear/utils.py: the
tensor-parallel region functions (defined in ``scaling_b200.parallel.collectives``) and the device choice of a layer."""

from __future__ import annotations

from typing import Any, Optional

import torch

from ....parallel.collectives import (  # noqa: F401
    all_concat,
    all_reduce,
    all_reduce_scatter_to_sequence_parallel,
    all_shard,
    copy_to_tensor_model_parallel_region,
    gather_from_sequence_parallel_region,
)


def get_device(topology: Optional[Any] = None, device: Optional[torch.device] = None) -> torch.device:
    """Where a layer puts its parameters: the topology's device, else the given one, else the current CUDA device
    (the CPU on a machine without one).  Naming both is an error."""
    assert topology is None or device is None, "cannot specify both device and topology"
    if topology is not None:
        return topology.device
    if device is not None:
        return device
    try:
        return torch.device(type="cuda", index=torch.cuda.current_device())
    except Exception:  # noqa: BLE001
        return torch.device("cpu")
