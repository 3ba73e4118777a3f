"""Configuration tree of the transformer application.

Field names, defaults and derived behaviour follow the reference
(src/scaling/transformer/context/config.py:28-635) so that its YAML files load unchanged: the legacy
key ``luminous_architecture`` is accepted, and ``trainer.separate_file_for_parameters`` is derived
from the names of the bitfit / adapter / softprompt fine-tuning components.
"""

from __future__ import annotations

from copy import deepcopy
from enum import Enum
from pathlib import Path
from typing import Any, List, Literal, Mapping, Optional, Union

import torch
from pydantic import Field, model_validator

from ...core.config import BaseConfig
from ...core.data.blended_dataset_config import BlendedDatasetConfig
from ...core.fp8 import FP8LinearConfig
from ...core.logging import LoggerConfig
from ...core.nn.attention import RelativePositionEmbeddingType
from ...core.nn.lora import LoRaConfig
from ...core.nn.masked_softmax import MaskedSoftmaxConfig
from ...core.nn.norm import LayerNormConfig, NormType
from ...core.optimizer import LearningRateSchedulerConfig, OptimizerConfig
from ...core.profiler import ProfilerConfig
from ...core.runner import RunnerConfig
from ...core.trainer import TrainerConfig
from ...parallel.topology_config import TopologyConfig


class Precision(Enum):
    FLOAT16 = "float16"
    BFLOAT16 = "bfloat16"
    FLOAT32 = "float32"

    @property
    def dtype(self) -> torch.dtype:
        return {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}[self.value]


class MLPType(Enum):
    DEFAULT = "default"
    SWIGLU = "swiglu"


class LossFunctionType(str, Enum):
    CROSS_ENTROPY_LOSS = "cross_entropy_loss"
    CONTRASTIVE_LOSS = "contrastive_loss"


class BaseLossFunctionConfig(BaseConfig):
    loss_type: LossFunctionType = Field(description="type of loss function")


class CrossEntropyLossFunctionConfig(BaseLossFunctionConfig):
    loss_type: Literal[LossFunctionType.CROSS_ENTROPY_LOSS] = Field(LossFunctionType.CROSS_ENTROPY_LOSS)


class ContrastiveLossFunctionConfig(BaseLossFunctionConfig):
    loss_type: Literal[LossFunctionType.CONTRASTIVE_LOSS] = Field(LossFunctionType.CONTRASTIVE_LOSS)
    number_of_hard_negatives: int = Field(1, description="hard negatives per positive sample")
    use_instructions: bool = Field(True, description="prepend an instruction to the text to embed, if available")
    query_side_only: bool = Field(False, description="with instructions: only the query receives one")
    scale: int = Field(1, description="divide cosine scores by this factor")
    log_verbose_metrics: bool = Field(True, description="compute all embedding fine-tuning metrics, not just the loss")


class TrainingGroupConfig(BaseConfig):
    group_name: str = Field(description="name of the group")
    parameters_include: Optional[List[str]] = Field(None, description="regexes of parameters in this group")
    parameters_exclude: List[str] = Field([], description="regexes of parameters kept out of this group")
    weight_decay: float = Field(0.0001, description="decoupled weight decay")
    independent_weight_decay: bool = Field(False, description="decay independent of the learning rate")
    learning_rate_scheduler: LearningRateSchedulerConfig = Field(LearningRateSchedulerConfig(), description="schedule")

    @model_validator(mode="after")
    def _no_overlap(self) -> "TrainingGroupConfig":
        if self.parameters_include is not None:
            both = set(self.parameters_include) & set(self.parameters_exclude)
            if both:
                raise ValueError(
                    "No overlap is allowed between parameters_include and parameters_exclude. "
                    f"Found the following keys in both lists: {', '.join(sorted(both))}. "
                )
        return self


class TrainingConfig(BaseConfig):
    allow_missing_params_in_optimizer: bool = Field(
        False, description="allow parameters outside every training group (they stay frozen)"
    )
    use_deterministic_torch_algorithms: bool = Field(False, description="torch.use_deterministic_algorithms(True)")
    loss_function_config: Union[ContrastiveLossFunctionConfig, CrossEntropyLossFunctionConfig] = Field(
        CrossEntropyLossFunctionConfig(), description="loss used in training"
    )


class BitfitBiasConfig(BaseConfig):
    name: str = Field(description="name of the bias set (parameters are called bias_{name})")
    version: str = Field(".unknown.", description="version tag of the config")


class SoftpromptConfig(BaseConfig):
    name: str = Field(description="name of the soft prompt")
    n_tokens: int = Field(description="number of learned prompt tokens")
    version: str = Field(".unknown.", description="version tag of the config")


class AdapterConfig(BaseConfig):
    name: str = Field(description="name of the adapter set")
    attention_downsampling_factor: Optional[float] = Field(None, description="bottleneck factor after attention")
    mlp_downsampling_factor: Optional[float] = Field(None, description="bottleneck factor after the MLP")
    init_std: float = Field(1.0e-5, description="std of the adapter weight init")
    version: str = Field(".unknown.", description="version tag of the config")


class PoolingMethod(str, Enum):
    MEAN = "mean"
    WEIGHTED_MEAN = "weighted_mean"
    LAST_TOKEN = "last_token"


class EmbeddingHeadConfig(BaseConfig):
    name: str = Field(description="name of the embedding head")
    proj_layers: Optional[List[int]] = Field(description="widths of the projection layers")
    pooling: PoolingMethod = Field(default=PoolingMethod.WEIGHTED_MEAN, description="token pooling")


class UMuPConfig(BaseConfig):
    enable: bool = Field(False, description="enables u-mup")
    allow_non_umup_params: bool = Field(False, description="tolerate parameters without u-mup meta")
    normalize_depth_to_num_layers: bool = Field(False, description="use num_layers as depth instead of residual count")
    attn_mult: float = Field(1.0, description="attention softmax temperature")
    act_mult: float = Field(1.0, description="temperature for mlp nonlinearity")
    residual_mult: float = Field(1.0, description="overall residual strength")
    residual_attn_ratio: float = Field(1.0, description="ratio of attn to mlp residual strength")
    loss_mult: float = Field(1.0, description="cross-entropy softmax temperature")


class TransformerArchitectureConfig(BaseConfig):
    vocab_size: int = Field(0, description="size of the vocabulary")
    vocab_file: Optional[Path] = Field(None, description="tokenizer file copied into checkpoints")
    hidden_size: int = Field(0, description="width of the residual stream")
    num_layers: int = Field(0, description="number of transformer layers")
    num_attention_heads: int = Field(0, description="number of query heads")
    num_local_attention_heads: int = Field(0, description="heads restricted to a sliding window")
    local_attention_window_size: Optional[int] = Field(None, description="size of the local attention window")
    rotary_embedding_base: int = Field(10000, description="base of the rotary frequencies")
    rotary_percentage: float = Field(1.0, description="fraction of each head that is rotated")
    sequence_length: int = Field(2048, description="training sequence length")
    norm_type: NormType = Field(NormType.LAYERNORM, description="layernorm or rms")
    relative_position_embedding_type: RelativePositionEmbeddingType = Field(
        RelativePositionEmbeddingType.ROTARY, description="none, rotary (rotate-half) or rotary_complex (interleaved)"
    )
    mlp_type: MLPType = Field(MLPType.DEFAULT, description="default (GELU) or swiglu")
    mlp_factor: float = Field(4.0, description="intermediate width / hidden size")
    attention_bias: bool = Field(True, description="bias in the attention projections")
    attention_qkv_in_one: bool = Field(True, description="one fused QKV projection (needs equal head counts)")
    attention_num_kv_heads: Optional[int] = Field(None, description="KV heads for GQA / MQA")
    attention_use_matmul: bool = Field(False, description="kept for config compatibility")
    reset_attention_mask: bool = Field(True, description="resets the attention mask between documents in a sequence")
    reset_position_ids: bool = Field(True, description="resets the position ids between documents in a sequence")
    mlp_bias: bool = Field(True, description="bias in the MLP projections")
    key_query_norm: bool = Field(False, description="per-head norm of queries and keys")
    weight_tying: bool = Field(True, description="share the embedding with the LM head")
    masked_softmax: MaskedSoftmaxConfig = Field(MaskedSoftmaxConfig(), description="attention kernel selection")
    layernorm: LayerNormConfig = Field(LayerNormConfig(), description="norm settings")
    precision: Precision = Field(Precision.FLOAT32, description="parameter / activation dtype")
    fp8_config_attention: Optional[FP8LinearConfig] = Field(None, description="fp8 for the QKV projections")
    fp8_config_attention_dense_out: Optional[FP8LinearConfig] = Field(None, description="fp8 for attention dense")
    fp8_config_mlp: Optional[FP8LinearConfig] = Field(None, description="fp8 for the MLP input projections")
    fp8_config_mlp_dense_out: Optional[FP8LinearConfig] = Field(None, description="fp8 for the MLP output projection")
    fp8_config_lm_head: Optional[FP8LinearConfig] = Field(None, description="fp8 for the LM head")
    dropout_embedding: float = Field(0.0, description="dropout applied after the embedding layer", ge=0.0, le=1.0)
    dropout_attention_probs: float = Field(0.0, description="dropout on attention probabilities", ge=0.0, le=1.0)
    dropout_after_attention: float = Field(0.0, description="dropout after the attention block", ge=0.0, le=1.0)
    dropout_after_mlp: float = Field(0.0, description="dropout after the MLP block", ge=0.0, le=1.0)
    bitfit_bias_config: Optional[BitfitBiasConfig] = Field(None, description="train a separate set of biases")
    finetunable_token_ids: List[int] = Field([], description="token ids whose embeddings receive gradients")
    image_encoder: bool = Field(False, description="add the CLIP image encoder to the input embedding")
    dropout_image_encoder: float = Field(0.0, description="dropout after the image encoder", ge=0.0, le=1.0)
    softprompt_config: Optional[SoftpromptConfig] = Field(None, description="learned prompt tokens")
    adapter_config: Optional[AdapterConfig] = Field(None, description="bottleneck adapters")
    lora_config: Optional[LoRaConfig] = Field(None, description="creates LoRa finetuning configuration")
    embedding_head_config: Optional[EmbeddingHeadConfig] = Field(None, description="pooled embedding head")
    lm_head: bool = Field(True, description="attach the language-model head")
    causal: bool = Field(True, description="Make attention layers causal.")
    umup: UMuPConfig = Field(UMuPConfig(), description="u-mup settings")

    @model_validator(mode="after")
    def _checks(self) -> "TransformerArchitectureConfig":
        if self.attention_num_kv_heads is not None and self.attention_qkv_in_one:
            if self.attention_num_kv_heads != self.num_attention_heads:
                raise ValueError("attention_num_kv_heads requires attention_qkv_in_one: false")
        return self


class DataConfig(BaseConfig):
    legacy_dataset: bool = Field(False, description="read Megatron indexed datasets")
    load_mmap_index_to_memory: bool = Field(False, description="hold the document index in memory")
    use_mmap: bool = Field(True, description="mmap reads (false: retryable file reads)")
    load_data_item_mmap_index_to_memory: bool = Field(False, description="hold the data-item index in memory")
    finetuning_dataset: bool = Field(False, description="prompt / completion jsonl data")
    finetuning_chat_dataset: bool = Field(False, description="chat jsonl data")
    finetuning_dataset_memory_map: bool = Field(False, description="fine-tuning data stored as memory map")
    embedding_dataset: bool = Field(False, description="query / positive / negatives data")
    embedding_dataset_memory_map: bool = Field(False, description="embedding data stored as memory map")
    data_prefixes: Optional[List[Path]] = Field(None, description="training data prefixes")
    validation_data_prefixes: Optional[List[Path]] = Field(None, description="validation data prefixes")
    blended_dataset: BlendedDatasetConfig = Field(BlendedDatasetConfig(), description="blending of several datasets")
    only_full_sequences: bool = Field(False, description="skip document tails that cannot fill a whole sequence")
    allow_incomplete_sequences_every_n: int = Field(0, description="with only_full_sequences: keep every n-th tail")
    synthetic_samples: Optional[int] = Field(
        None, description="if set and no data_prefixes are given: this many seeded uniform-random sequences"
    )


def is_legacy_config(config: Mapping[str, Any]) -> bool:
    return "luminous_architecture" in config


def convert_legacy_config(config: Mapping[str, Any]) -> dict[str, Any]:
    new = dict(config)
    new["transformer_architecture"] = new.pop("luminous_architecture")
    return new


class TransformerConfig(BaseConfig):
    version: str = Field(".unknown.", description="version tag of the config")
    runner: RunnerConfig = Field(RunnerConfig(), description="launcher settings")
    logger: LoggerConfig = Field(LoggerConfig(), description="logging settings")
    topology: TopologyConfig = Field(
        TopologyConfig(model_parallel_size=1, pipe_parallel_size=1, data_parallel_size=1, micro_batch_size=2,
                       gradient_accumulation_steps=1),  # type: ignore[call-arg]
        description="parallel layout and batch sizes (default: one process, micro batch 2)",
    )
    optimizer: OptimizerConfig = Field(OptimizerConfig(), description="optimizer settings")
    training: TrainingConfig = Field(TrainingConfig(), description="training settings")
    training_groups: List[TrainingGroupConfig] = Field(default=[], description="parameter groups by regex")
    trainer: TrainerConfig = Field(TrainerConfig(), description="trainer settings")
    profiler: ProfilerConfig = Field(ProfilerConfig(), description="profiler settings")
    transformer_architecture: TransformerArchitectureConfig = Field(
        TransformerArchitectureConfig(), description="model architecture"
    )
    data: DataConfig = Field(DataConfig(), description="dataset settings")
    determined_experiment_id: Optional[int] = Field(None, description="set by the Determined integration")
    determined_trial_id: Optional[int] = Field(None, description="set by the Determined integration")

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], overwrite_values: Optional[dict] = None) -> "TransformerConfig":
        d = deepcopy(dict(convert_legacy_config(d) if is_legacy_config(d) else d))
        arch = d.get("transformer_architecture") or {}
        separate = set()
        for key, prefix in (("bitfit_bias_config", "bias"), ("adapter_config", "adapter"),
                            ("softprompt_config", "softprompt")):
            if arch.get(key) is not None:
                separate.add(f"{prefix}_{arch[key]['name']}")
        if separate:
            d.setdefault("trainer", {})["separate_file_for_parameters"] = sorted(separate)
        return super().from_dict(d, overwrite_values=overwrite_values)

    @model_validator(mode="after")
    def _unique_group_names(self) -> "TransformerConfig":
        names = [g.group_name for g in self.training_groups]
        dup = {n for n in names if names.count(n) > 1}
        if dup:
            raise ValueError(
                f"Please give each training parameter group a unique name.\n"
                f"The following names showed up more than one time: {dup}"
            )
        return self
