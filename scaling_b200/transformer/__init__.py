from .context import TransformerArchitectureConfig, TransformerConfig, TransformerContext
from .data import (EmbeddingBlendedDataset, EmbeddingDataset, FinetuningChatBlendedDataset, FinetuningChatDataset,
                   FinetuningTextBlendedDataset, FinetuningTextDataset, LegacyBlendedDataset, SyntheticTextDataset,
                   TextBlendedDataset, TextDataset, TextDatasetBatch, TextDatasetItem, TextImageBlendedDataset,
                   TextImageDataset)
from .model import TransformerLayerIO, TransformerParallelModule, init_model, init_optimizer

__all__ = ["EmbeddingBlendedDataset", "EmbeddingDataset", "FinetuningChatBlendedDataset", "FinetuningChatDataset",
           "FinetuningTextBlendedDataset", "FinetuningTextDataset", "LegacyBlendedDataset", "SyntheticTextDataset",
           "TextBlendedDataset", "TextDataset", "TextDatasetBatch", "TextDatasetItem", "TextImageBlendedDataset",
           "TextImageDataset", "TransformerArchitectureConfig", "TransformerConfig", "TransformerContext",
           "TransformerLayerIO", "TransformerParallelModule", "init_model", "init_optimizer"]
