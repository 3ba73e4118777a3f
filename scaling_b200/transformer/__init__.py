from .context import TransformerArchitectureConfig, TransformerConfig, TransformerContext
from .data import SyntheticTextDataset, TextDataset, TextDatasetBatch, TextDatasetItem
from .model import TransformerLayerIO, TransformerParallelModule, init_model, init_optimizer

__all__ = ["SyntheticTextDataset", "TextDataset", "TextDatasetBatch", "TextDatasetItem", "TransformerArchitectureConfig",
           "TransformerConfig", "TransformerContext", "TransformerLayerIO", "TransformerParallelModule", "init_model",
           "init_optimizer"]
