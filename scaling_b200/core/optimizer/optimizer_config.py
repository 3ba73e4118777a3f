"""Optimizer settings (fields of src/scaling/core/optimizer/optimizer_config.py:7-42 and
parameter_group_config.py:9-29)."""

from __future__ import annotations

from typing import Optional

from pydantic import Field

from ..config import BaseConfig
from .learning_rate_scheduler import LearningRateSchedulerConfig
from .loss_scaler import LossScalerConfig


class OptimizerConfig(BaseConfig):
    method: str = Field("adamw", description="optimisation method (adamw)")
    beta1: float = Field(0.9, description="decay of the running average of the gradient")
    beta2: float = Field(0.95, description="decay of the running average of the squared gradient")
    eps: float = Field(1e-8, description="term added to the denominator for numerical stability")
    gradient_clipping: float = Field(1.0, description="clip the global l2 gradient norm to this value; 0 disables", ge=0.0)
    allreduce_bucket_size: int = Field(500000000, description="elements per collective bucket", gt=0)
    loss_scaler: LossScalerConfig = Field(LossScalerConfig(), description="dynamic loss scaling (fp16)")
    zero: bool = Field(False, description="shard optimizer states over data-parallel ranks (ZeRO stage 1)")
    zero_save_static: bool = Field(
        False, description="with zero: write each rank's raw optimizer state instead of layout-independent files"
    )
    debug_log: bool = Field(False, description="report per-parameter norms every step (slow)")
    fused_collectives: bool = Field(
        True, description="use the in-kernel NVLink reduce-scatter / all-gather when the group supports peer memory"
    )


class OptimizerParamGroupConfig(BaseConfig):
    name: Optional[str] = Field(None, description="name of the group in logs")
    learning_rate_scheduler: LearningRateSchedulerConfig = Field(
        LearningRateSchedulerConfig(), description="learning-rate schedule of the group"
    )
    weight_decay: float = Field(1e-2, description="decoupled weight decay")
    independent_weight_decay: bool = Field(
        False, description="decay by weight_decay alone instead of learning_rate * weight_decay"
    )
