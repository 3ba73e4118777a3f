"""Datasets from the ``data`` section of a transformer config (src/scaling/transformer/dataset_loader.py:19-172 and
the blending step of src/scaling/transformer/train.py:229-262).

``load_datasets`` returns one dataset per prefix for training and for validation; ``load_blended_datasets`` wraps
each list into the blended dataset class of its kind.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Optional, Sequence

from ..core.data import BaseDataset
from ..core.data.blended_dataset import BaseBlendedDataset
from .context.config import ContrastiveLossFunctionConfig, DataConfig, TransformerArchitectureConfig, TransformerConfig
from .data.text_dataset import TextDataset
from .tokenizer import Tokenizer, load_tokenizers


def _load_tokenizer(architecture: TransformerArchitectureConfig) -> tuple[Tokenizer, Tokenizer]:
    assert architecture.vocab_file is not None, "vocab_file needs to be set to load the vocabulary file."
    return load_tokenizers(architecture.vocab_file)


def _softprompt_n_tokens(architecture: TransformerArchitectureConfig) -> int:
    return 0 if architecture.softprompt_config is None else architecture.softprompt_config.n_tokens


def _text_datasets(prefixes: Sequence[Path], config: TransformerConfig) -> list[BaseDataset]:
    d, a = config.data, config.transformer_architecture
    return [
        TextDataset(data_prefix=p, sequence_length=a.sequence_length, seed=config.trainer.seed,
                    legacy_dataset=d.legacy_dataset, load_mmap_index_to_memory=d.load_mmap_index_to_memory,
                    load_data_item_mmap_index_to_memory=d.load_data_item_mmap_index_to_memory,
                    only_full_sequences=d.only_full_sequences,
                    allow_incomplete_sequences_every_n=d.allow_incomplete_sequences_every_n, use_mmap=d.use_mmap,
                    reset_attention_mask=a.reset_attention_mask, reset_position_ids=a.reset_position_ids)
        for p in prefixes
    ]


def _finetuning_text_datasets(prefixes: Sequence[Path], config: TransformerConfig) -> list[BaseDataset]:
    from .data.finetuning_text_dataset import FinetuningTextDataset

    a = config.transformer_architecture
    assert config.data.use_mmap, "Finetuning is currently only supported with use_mmap set to true."
    tok, tok_nps = _load_tokenizer(a)
    return [
        FinetuningTextDataset(data_prefix=p, sequence_length=a.sequence_length, seed=config.trainer.seed,
                              softprompt_n_tokens=_softprompt_n_tokens(a), tokenizer=tok,
                              tokenizer_no_prefix_space=tok_nps,
                              memory_map_dataset=config.data.finetuning_dataset_memory_map)
        for p in prefixes
    ]


def _finetuning_chat_datasets(prefixes: Sequence[Path], config: TransformerConfig) -> list[BaseDataset]:
    from .data.finetuning_chat_dataset import FinetuningChatDataset

    a = config.transformer_architecture
    tok, tok_nps = _load_tokenizer(a)
    return [
        FinetuningChatDataset(data_path=p, sequence_length=a.sequence_length, seed=config.trainer.seed,
                              softprompt_n_tokens=_softprompt_n_tokens(a), tokenizer=tok,
                              tokenizer_no_prefix_space=tok_nps)
        for p in prefixes
    ]


def _embedding_datasets(prefixes: Sequence[Path], config: TransformerConfig) -> list[BaseDataset]:
    from .data.embedding_dataset import EmbeddingDataset

    a = config.transformer_architecture
    loss = config.training.loss_function_config
    assert isinstance(loss, ContrastiveLossFunctionConfig), "embedding datasets go with the contrastive loss"
    tok, _ = _load_tokenizer(a)
    return [
        EmbeddingDataset(data_path=p, tokenizer=tok, memory_map_dataset=config.data.embedding_dataset_memory_map,
                         use_instruction=loss.use_instructions, number_of_hard_negatives=loss.number_of_hard_negatives,
                         sequence_length=a.sequence_length, seed=config.trainer.seed,
                         query_side_only=loss.query_side_only)
        for p in prefixes
    ]


def _maker(data_config: DataConfig):
    if data_config.finetuning_dataset:
        return _finetuning_text_datasets
    if data_config.finetuning_chat_dataset:
        return _finetuning_chat_datasets
    if data_config.embedding_dataset:
        return _embedding_datasets
    return _text_datasets


def load_datasets(data_config: DataConfig, architecture_config: TransformerArchitectureConfig,
                  config: TransformerConfig) -> tuple[Sequence[BaseDataset], Sequence[BaseDataset]]:
    """``(training datasets, validation datasets)``, one per configured prefix."""
    assert data_config.data_prefixes is not None, "path to data prefix not defined in Transformer context"
    make = _maker(data_config)
    train = make(data_config.data_prefixes, config)
    validation = make(data_config.validation_data_prefixes, config) if data_config.validation_data_prefixes else []
    return train, validation


def blended_dataset_type(data_config: DataConfig) -> type[BaseBlendedDataset]:
    if data_config.finetuning_dataset:
        from .data.finetuning_text_dataset import FinetuningTextBlendedDataset

        return FinetuningTextBlendedDataset
    if data_config.finetuning_chat_dataset:
        from .data.finetuning_chat_dataset import FinetuningChatBlendedDataset

        return FinetuningChatBlendedDataset
    if data_config.embedding_dataset:
        from .data.embedding_dataset import EmbeddingBlendedDataset

        return EmbeddingBlendedDataset
    from .data.legacy_blended_dataset import LegacyBlendedDataset
    from .data.text_dataset import TextBlendedDataset

    return LegacyBlendedDataset if data_config.legacy_dataset else TextBlendedDataset


def load_blended_datasets(config: TransformerConfig) -> tuple[BaseDataset, Optional[BaseDataset]]:
    """The training and (if configured) validation data of a run as single blended datasets."""
    train, validation = load_datasets(config.data, config.transformer_architecture, config)
    kind: Any = blended_dataset_type(config.data)
    seed = config.trainer.seed
    blended = kind(seed=seed, config=config.data.blended_dataset, datasets=train)
    blended_validation = None
    if validation:
        blended_validation = kind(seed=seed, config=config.data.blended_dataset, datasets=validation)
    return blended, blended_validation
