"""Layout of a job: sizes of the three parallel axes and the batch triple.

Mirrors the fields and the inference rules of the reference
(src/scaling/core/topology/topology_config.py:20-206): any three of
{model, pipe, data parallel size, world size} determine the fourth, any two of
{global batch, micro batch, gradient accumulation steps} determine the third, and
``global = micro * grad_acc * dp`` is always asserted.  Two fields are added for this build:
``backend`` (``nccl`` on GPUs, ``gloo`` for CPU ranks) and ``device`` (``cuda`` | ``cpu``).
"""

from __future__ import annotations

from enum import Enum
from typing import Any, List, Optional

from pydantic import Field, model_validator

from ..core.config import BaseConfig


class PipePartitionMethod(Enum):
    UNIFORM = "uniform"
    BALANCED = "balanced"


class ActivationCheckpointingType(Enum):
    EVERY_PIPE_STAGE = "every_pipe_stage"
    EVERY_LAYER = "every_layer"
    DISABLED = "disabled"


def _fill_parallel_sizes(mp, pp, dp, world):
    given = [v for v in (mp, pp, dp, world) if v is not None]
    if len(given) < 3:
        raise AssertionError(
            "At least 3 out of 4 parallelization parameters (model_parallel_size, pipe_parallel_size, "
            "data_parallel_size and world_size) need to be set."
        )
    if world is None:
        world = mp * pp * dp
    if mp is None:
        mp = world // (pp * dp)
    if pp is None:
        pp = world // (mp * dp)
    if dp is None:
        dp = world // (mp * pp)
    assert mp >= 1 and pp >= 1 and dp >= 1 and mp * pp * dp == world, (
        f"world_size {world} does not equal the product of model_parallel_size ({mp}), pipe_parallel_size ({pp}) "
        f"and data_parallel_size ({dp})."
    )
    return mp, pp, dp, world


def _fill_batch_sizes(global_bs, micro_bs, grad_acc, dp):
    given = [v for v in (global_bs, micro_bs, grad_acc) if v is not None]
    if len(given) < 2:
        raise AssertionError(
            "At least 2 out of 3 batch size parameters (global_batch_size, micro_batch_size, "
            "and gradient_accumulation_steps) need to be set."
        )
    if grad_acc is None:
        grad_acc = global_bs // (micro_bs * dp)
    if micro_bs is None:
        micro_bs = global_bs // (grad_acc * dp)
    if global_bs is None:
        global_bs = micro_bs * grad_acc * dp
    assert global_bs == micro_bs * grad_acc * dp, (
        f"global_batch_size {global_bs} does not equal the product of micro_batch_size ({micro_bs}) "
        f"and gradient_accumulation_steps ({grad_acc}) and data_parallel_size ({dp})."
    )
    return global_bs, micro_bs, grad_acc


class TopologyConfig(BaseConfig):
    global_rank: Optional[int] = Field(None, description="rank of this process in the job", ge=0)
    world_size: int = Field(description="number of processes (one per GPU)", gt=0)
    local_slot: Optional[int] = Field(None, description="device index on this node", ge=0)
    model_parallel_size: int = Field(description="tensor-parallel width", gt=0)
    pipe_parallel_size: int = Field(description="number of pipeline stages", gt=0)
    data_parallel_size: int = Field(description="number of model replicas", gt=0)
    global_batch_size: int = Field(description="samples per optimizer step over all replicas", gt=0)
    micro_batch_size: int = Field(description="samples per forward/backward pass of one replica", gt=0)
    gradient_accumulation_steps: int = Field(description="micro batches per optimizer step", gt=0)
    pipe_partition_method: PipePartitionMethod = Field(
        PipePartitionMethod.UNIFORM, description="how layers are assigned to pipeline stages"
    )
    pipe_partition_overwrite: Optional[List[int]] = Field(None, description="explicit stage boundaries")
    activation_checkpointing_type: ActivationCheckpointingType = Field(
        ActivationCheckpointingType.DISABLED, description="recompute granularity"
    )
    sequence_parallel: bool = Field(False, description="shard the residual stream over tokens inside a TP group")
    backend: Optional[str] = Field(None, description="torch.distributed backend; default nccl on cuda, gloo on cpu")
    device: Optional[str] = Field(None, description="'cuda' or 'cpu'; default cuda when available")

    @model_validator(mode="before")
    @classmethod
    def _infer_sizes(cls, values: Any) -> Any:
        if not isinstance(values, dict):
            return values
        values = dict(values)
        mp, pp, dp, world = _fill_parallel_sizes(
            values.get("model_parallel_size"),
            values.get("pipe_parallel_size"),
            values.get("data_parallel_size"),
            values.get("world_size"),
        )
        gbs, mbs, ga = _fill_batch_sizes(
            values.get("global_batch_size"),
            values.get("micro_batch_size"),
            values.get("gradient_accumulation_steps"),
            dp,
        )
        values.update(
            world_size=world,
            model_parallel_size=mp,
            pipe_parallel_size=pp,
            data_parallel_size=dp,
            global_batch_size=gbs,
            micro_batch_size=mbs,
            gradient_accumulation_steps=ga,
        )
        values.setdefault("global_rank", None)
        return values
