"""Configuration tree of the MLP classifier application (the complete small example on the core API;
counterpart of examples/mlp_example/config.py in the reference)."""

from __future__ import annotations

from pathlib import Path
from typing import Optional

from pydantic import Field

from ...core.config import BaseConfig
from ...core.logging import LoggerConfig
from ...core.optimizer import LearningRateSchedulerConfig, OptimizerConfig
from ...core.profiler import ProfilerConfig
from ...core.runner import RunnerConfig
from ...core.trainer import TrainerConfig
from ...parallel.topology_config import TopologyConfig


class MLPArchitectureConfig(BaseConfig):
    n_hidden_layers: int = Field(1, description="hidden layers between the input and the output projection")
    hidden_dim: int = Field(256, description="width of the hidden layers")
    input_dim: int = Field(784, description="flattened input size")
    output_dim: int = Field(10, description="number of classes")
    precision: str = Field("float32", description="parameter dtype: float32, bfloat16 or float16")


class MLPTrainingConfig(BaseConfig):
    weight_decay: float = Field(0.0001, description="decoupled weight decay")


class MLPDataConfig(BaseConfig):
    synthetic: bool = Field(True, description="uniform random inputs / labels from a seed instead of image files")
    n_samples: int = Field(4096, description="size of the synthetic dataset")
    mnist_dir: Optional[Path] = Field(None, description="directory with MNIST idx files (no download is attempted)")


class MLPConfig(BaseConfig):
    runner: RunnerConfig = Field(RunnerConfig(), description="launcher settings")
    logger: LoggerConfig = Field(LoggerConfig(), description="logging settings")
    topology: TopologyConfig = Field(description="parallel layout and batch sizes")
    optimizer: OptimizerConfig = Field(OptimizerConfig(), description="optimizer settings")
    learning_rate_scheduler: LearningRateSchedulerConfig = Field(LearningRateSchedulerConfig(), description="schedule")
    training: MLPTrainingConfig = Field(MLPTrainingConfig(), description="training settings")
    trainer: TrainerConfig = Field(TrainerConfig(), description="trainer settings")
    profiler: ProfilerConfig = Field(ProfilerConfig(), description="profiler settings")
    architecture: MLPArchitectureConfig = Field(MLPArchitectureConfig(), description="model shape")
    data: MLPDataConfig = Field(MLPDataConfig(), description="dataset settings")
