from .inference_settings import Control, InferenceSettings, InferenceSuppressionParameters
from .text_dataset import SyntheticTextDataset, TextDataset, TextDatasetItem, pack_windows
from .text_dataset_batch import TextDatasetBatch, TextDatasetBatchBeforeSync
from .utils import (
    add_cumulative_seq_lengths_padding,
    document_ranges_from_padded,
    get_cumulative_seq_lengths,
    get_cumulative_seq_lengths_padded,
    get_position_ids,
    remove_cumulative_seq_lengths_padding,
)

__all__ = ["Control", "InferenceSettings", "InferenceSuppressionParameters", "SyntheticTextDataset", "TextDataset",
           "TextDatasetBatch", "TextDatasetBatchBeforeSync", "TextDatasetItem", "add_cumulative_seq_lengths_padding", "document_ranges_from_padded", "get_cumulative_seq_lengths_padded",
           "get_cumulative_seq_lengths", "get_position_ids", "pack_windows", "remove_cumulative_seq_lengths_padding"]
