from .dataset_item import TextImageDatasetItem
from .embedding_dataset import EmbeddingBlendedDataset, EmbeddingDataset, EmbeddingDatasetItem
from .finetuning_chat_dataset import FinetuningChatBlendedDataset, FinetuningChatDataset
from .finetuning_text_dataset import FinetuningTextBlendedDataset, FinetuningTextDataset
from .inference_settings import Control, InferenceSettings, InferenceSuppressionParameters
from .legacy_blended_dataset import LegacyBlendedDataset
from .text_dataset import SyntheticTextDataset, TextBlendedDataset, TextDataset, TextDatasetItem, pack_windows
from .text_image_dataset import TextImageBlendedDataset, TextImageDataset
from .text_dataset_batch import TextDatasetBatch, TextDatasetBatchBeforeSync
from .utils import (
    add_cumulative_seq_lengths_padding,
    document_ranges_from_padded,
    get_cumulative_seq_lengths,
    get_cumulative_seq_lengths_padded,
    get_position_ids,
    remove_cumulative_seq_lengths_padding,
)

__all__ = ["EmbeddingBlendedDataset", "EmbeddingDataset", "EmbeddingDatasetItem", "FinetuningChatBlendedDataset",
           "FinetuningChatDataset", "FinetuningTextBlendedDataset", "FinetuningTextDataset", "TextBlendedDataset",
           "TextImageDatasetItem", "TextImageBlendedDataset", "TextImageDataset", "LegacyBlendedDataset", "Control", "InferenceSettings", "InferenceSuppressionParameters", "SyntheticTextDataset", "TextDataset",
           "TextDatasetBatch", "TextDatasetBatchBeforeSync", "TextDatasetItem", "add_cumulative_seq_lengths_padding", "document_ranges_from_padded", "get_cumulative_seq_lengths_padded",
           "get_cumulative_seq_lengths", "get_position_ids", "pack_windows", "remove_cumulative_seq_lengths_padding"]
