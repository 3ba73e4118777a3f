"""Public surface of the engine (the names exported by src/scaling/core/__init__.py).

Names are resolved on first access (PEP 562): the engine's subpackages and ``scaling_b200.parallel`` import each
other's configuration classes, so nothing is imported here at package import time."""

from __future__ import annotations

import importlib
from typing import Any

_EXPORTS = {
    "ActivationFunction": ".nn.mlp",
    "BaseBlendedDataset": ".data",
    "BaseConfig": ".config",
    "BaseContext": ".context",
    "BaseContextGeneric": ".context",
    "BaseDataset": ".data",
    "BaseDatasetBatch": ".data",
    "BaseDatasetItem": ".data",
    "BaseLayer": ".nn.parallel_module",
    "BaseLayerIO": ".data",
    "BaseOptimizer": ".optimizer",
    "BaseTrainer": ".trainer",
    "BlendedDatasetConfig": ".data",
    "ColumnParallelLinear": ".nn.linear",
    "CoreParameterMeta": ".nn.parameter_meta",
    "DataLoader": ".data",
    "DeterminedBaseContext": ".context",
    "DeterminedBaseTrainer": ".trainer",
    "FileDataset": ".data",
    "LayerNorm": ".nn.norm",
    "LayerNormConfig": ".nn.norm",
    "LayerNormOptimizationType": ".nn.norm",
    "LayerSpec": ".nn.parallel_module",
    "LearningRateDecayStyle": ".optimizer",
    "LearningRateScheduler": ".optimizer",
    "LearningRateSchedulerConfig": ".optimizer",
    "LoRAModuleType": ".nn.lora",
    "LoRaConfig": ".nn.lora",
    "LossScaler": ".optimizer",
    "LossScalerConfig": ".optimizer",
    "MaskedSoftmax": ".nn.masked_softmax",
    "MaskedSoftmaxConfig": ".nn.masked_softmax",
    "MaskedSoftmaxKernel": ".nn.masked_softmax",
    "MemoryMapDataset": ".data",
    "MemoryMapDatasetBuilder": ".data",
    "NormType": ".nn.norm",
    "Optimizer": ".optimizer",
    "OptimizerConfig": ".optimizer",
    "OptimizerParamGroup": ".optimizer",
    "OptimizerParamGroupConfig": ".optimizer",
    "ParallelLoRa": ".nn.lora",
    "ParallelMLP": ".nn.mlp",
    "ParallelModule": ".nn.parallel_module",
    "ParallelSelfAttention": ".nn.attention",
    "ParallelSwiGLUMLP": ".nn.mlp",
    "PipePartitionCoordinates": ".nn.parallel_module",
    "PipePartitionMethod": "..parallel",
    "PipelineScheduleInference": ".nn.pipeline_schedule",
    "PipelineScheduleTrain": ".nn.pipeline_schedule",
    "Profiler": ".profiler",
    "ProfilerConfig": ".profiler",
    "RMSNorm": ".nn.norm",
    "RelativePositionEmbeddingType": ".nn.attention",
    "RotaryConfig": ".nn.rotary",
    "RotaryEmbedding": ".nn.rotary",
    "RotaryEmbeddingComplex": ".nn.rotary",
    "RowParallelLinear": ".nn.linear",
    "RunnerConfig": ".runner",
    "RunnerDockerConfig": ".runner",
    "RunnerType": ".runner",
    "SynchronizedTimer": ".profiler",
    "TiedLayerSpec": ".nn.parallel_module",
    "Topology": "..parallel",
    "TopologyConfig": "..parallel",
    "TrainerConfig": ".trainer",
    "VocabParallelEmbedding": ".nn.linear",
    "broadcast_data": ".data",
    "get_activation_function": ".nn.mlp",
    "get_norm": ".nn.norm",
    "pipe_partition_uniform": ".nn.parallel_module",
    "runner_main": ".runner",
}

__all__ = sorted(_EXPORTS)


def __getattr__(name: str) -> Any:
    target = _EXPORTS.get(name)
    if target is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(importlib.import_module(target, __name__), name)
    globals()[name] = value
    return value


def __dir__() -> list[str]:
    return sorted(list(globals()) + list(_EXPORTS))
