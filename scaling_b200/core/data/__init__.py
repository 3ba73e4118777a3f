from .base_dataset import BaseDataset, BaseDatasetBatch, BaseDatasetItem
from .base_layer_io import BaseLayerIO
from .broadcast_data import broadcast_data
from .dataloader import DataLoader, RandomSampler
from .file_dataset import FileDataset
from .file_handles import FileHandle, RetryableException
from .memory_map import MemoryMapDataset, MemoryMapDatasetBuilder

__all__ = ["BaseDataset", "BaseDatasetBatch", "BaseDatasetItem", "BaseLayerIO", "DataLoader", "FileDataset",
           "FileHandle", "MemoryMapDataset", "MemoryMapDatasetBuilder", "RandomSampler", "RetryableException",
           "broadcast_data"]
