"""Public surface of the engine (the names exported by src/scaling/core/__init__.py)."""

from ..parallel import PipePartitionMethod, Topology, TopologyConfig
from .config import BaseConfig
from .context import BaseContext, BaseContextGeneric, DeterminedBaseContext
from .data import (BaseBlendedDataset, BaseDataset, BaseDatasetBatch, BaseDatasetItem, BaseLayerIO, BlendedDatasetConfig,
                   DataLoader, FileDataset, MemoryMapDataset, MemoryMapDatasetBuilder, broadcast_data)
from .nn.attention import ParallelSelfAttention, RelativePositionEmbeddingType
from .nn.linear import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding
from .nn.lora import LoRAModuleType, LoRaConfig, ParallelLoRa
from .nn.masked_softmax import MaskedSoftmax, MaskedSoftmaxConfig, MaskedSoftmaxKernel
from .nn.mlp import ActivationFunction, ParallelMLP, ParallelSwiGLUMLP, get_activation_function
from .nn.norm import LayerNorm, LayerNormConfig, LayerNormOptimizationType, NormType, RMSNorm, get_norm
from .nn.parallel_module import (BaseLayer, LayerSpec, ParallelModule, PipePartitionCoordinates, TiedLayerSpec,
                                 pipe_partition_uniform)
from .nn.parameter_meta import CoreParameterMeta
from .nn.pipeline_schedule import PipelineScheduleInference, PipelineScheduleTrain
from .nn.rotary import RotaryConfig, RotaryEmbedding, RotaryEmbeddingComplex
from .optimizer import (BaseOptimizer, LearningRateDecayStyle, LearningRateScheduler, LearningRateSchedulerConfig,
                        LossScaler, LossScalerConfig, Optimizer, OptimizerConfig, OptimizerParamGroup,
                        OptimizerParamGroupConfig)
from .profiler import Profiler, ProfilerConfig, SynchronizedTimer
from .runner import RunnerConfig, RunnerDockerConfig, RunnerType, runner_main
from .trainer import BaseTrainer, DeterminedBaseTrainer, TrainerConfig

__all__ = [
    "ActivationFunction", "BaseBlendedDataset", "BaseConfig", "BaseContext", "BaseContextGeneric", "BaseDataset",
    "BaseDatasetBatch", "BaseDatasetItem", "BaseLayer", "BaseLayerIO", "BaseOptimizer", "BaseTrainer",
    "BlendedDatasetConfig", "ColumnParallelLinear", "CoreParameterMeta", "DataLoader", "DeterminedBaseContext",
    "DeterminedBaseTrainer", "FileDataset", "LayerNorm", "LayerNormConfig", "LayerNormOptimizationType", "LayerSpec",
    "LearningRateDecayStyle", "LearningRateScheduler", "LearningRateSchedulerConfig", "LoRAModuleType", "LoRaConfig",
    "LossScaler", "LossScalerConfig", "MaskedSoftmax", "MaskedSoftmaxConfig", "MaskedSoftmaxKernel", "MemoryMapDataset",
    "MemoryMapDatasetBuilder", "NormType", "Optimizer", "OptimizerConfig", "OptimizerParamGroup",
    "OptimizerParamGroupConfig", "ParallelLoRa", "ParallelMLP", "ParallelModule", "ParallelSelfAttention",
    "ParallelSwiGLUMLP", "PipePartitionCoordinates", "PipePartitionMethod", "PipelineScheduleInference",
    "PipelineScheduleTrain", "Profiler", "ProfilerConfig", "RMSNorm", "RelativePositionEmbeddingType", "RotaryConfig",
    "RotaryEmbedding", "RotaryEmbeddingComplex", "RowParallelLinear", "RunnerConfig", "RunnerDockerConfig",
    "RunnerType", "SynchronizedTimer", "TiedLayerSpec", "Topology", "TopologyConfig", "TrainerConfig",
    "VocabParallelEmbedding", "broadcast_data", "get_activation_function", "get_norm", "pipe_partition_uniform",
    "runner_main",
]
