"""Text + image examples from a protobuf memory map (src/scaling/transformer/data/text_image_dataset.py:31-408).

Records (``TextImageExample``) carry ready-made input / target token lists, a loss mask, the encoded image files and
the token ranges the images occupy.  An item is one record padded or cut to ``sequence_length``; the order of records
is a seeded permutation stored as an index cache next to the data (built by global rank 0, awaited by the others).
"""

from __future__ import annotations

import hashlib
import time
from io import BytesIO
from pathlib import Path
from typing import List, Optional, Union

import numpy as np
import torch
import torch.distributed as dist

from ...core.data import BaseDataset, FileDataset, MemoryMapDataset, MemoryMapDatasetBuilder
from ...core.data.blended_dataset import BaseBlendedDataset
from ...core.data.pb_memory_map import PbMemoryMap, TextImageExample
from ...core.logging import logger
from ...parallel.topology import Topology
from ._finetuning_common import collate_items, image_transform, shift_locations, sync_text_image_batch
from .dataset_item import TextImageDatasetItem
from .text_dataset_batch import TextDatasetBatch


class TextImageDataset(BaseDataset[TextImageDatasetItem, TextDatasetBatch, TextDatasetBatch]):
    def __init__(self, data_prefix: Path, sequence_length: int, softprompt_n_tokens: int,
                 data_index_prefix: Optional[Path] = None, padding_token_id: int = 0, shuffle: bool = True,
                 seed: int = 42, use_mmap: bool = True, load_data_item_mmap_index_to_memory: bool = False):
        self.data_path_parent = Path(data_prefix).parent
        self.sequence_length = sequence_length
        self.softprompt_n_tokens = softprompt_n_tokens
        self.padding_token_id = padding_token_id
        self.seed: Optional[int] = None
        self.data_item_index: Union[MemoryMapDataset, FileDataset, None] = None
        self.load_data_item_mmap_index_to_memory = load_data_item_mmap_index_to_memory
        self.use_mmap = use_mmap
        self.memory_map = PbMemoryMap(prefix_path=data_prefix, pb_datatype=TextImageExample)
        super().__init__(seed=seed, shuffle=shuffle, data_prefix=data_prefix, data_index_prefix=data_index_prefix)

    def ident(self) -> str:
        return f"{hashlib.md5(str(self.data_prefix).encode('utf-8')).hexdigest()}-seq-{self.sequence_length}"

    def set_seed(self, seed: int, shuffle: bool = True) -> None:
        if self.seed is not None and self.seed == seed:
            return
        self.seed = seed
        stem = self.get_data_index_cache_filename_stem(seed)
        files = [Path(self.get_data_index_cache_filename_bin(seed)), Path(self.get_data_index_cache_filename_idx(seed)),
                 Path(self.get_data_index_cache_filename_meta(seed))]
        builder_rank = not dist.is_initialized() or dist.get_rank() == 0
        if not files[2].is_file() and builder_rank:
            for f in files[:2]:
                f.unlink(missing_ok=True)
            order = np.arange(len(self.memory_map))
            if shuffle:
                np.random.RandomState(seed=seed).shuffle(order)
            builder = MemoryMapDatasetBuilder(Path(stem), dtype=np.dtype(np.int64), index_dtype=np.dtype(np.int64))
            for record in order:
                builder.add(np.array([record]))
            builder.finalize()
        waited = 0
        while not all(f.is_file() for f in files):
            waited += 1
            if waited % 12 == 0:
                logger.info(f"TextImageDataset waiting on index for seed {seed} for {Path(self.data_prefix).name}; "
                            f"elapsed {waited * 5 / 60:.1f} minutes")
            time.sleep(5)
        cls = MemoryMapDataset if self.use_mmap else FileDataset
        self.data_item_index = cls(prefix_path=Path(stem), load_index_to_memory=self.load_data_item_mmap_index_to_memory)

    def __len__(self) -> int:
        return len(self.memory_map)

    def __getitem__(self, index: int) -> TextImageDatasetItem:
        if self.data_item_index is None:
            raise ValueError("Data item index not set. Call 'set_seed' before accessing data.")
        rec = self.memory_map[int(self.data_item_index[index][0])]
        S, n_soft = self.sequence_length, self.softprompt_n_tokens
        inputs = [0] * n_soft + list(rec["input_token_list"])
        targets = [0] * n_soft + list(rec["target_token_list"])
        mask = [0] * n_soft + [int(m) for m in rec["loss_mask_list"]]
        locations = shift_locations([(loc["start_index"], loc["end_index"]) for loc in rec["prompt_image_locations"]],
                                    n_soft)
        fill = max(S - len(inputs), 0)
        inputs = (inputs + [self.padding_token_id] * fill)[:S]
        targets = (targets + [self.padding_token_id] * fill)[:S]
        mask = (mask + [0] * fill)[:S]
        images = []
        if rec["prompt_image_data"]:
            from PIL import Image

            images = [image_transform()(Image.open(BytesIO(blob))) for blob in rec["prompt_image_data"]]
        return TextImageDatasetItem(
            input_token_ids=torch.tensor(inputs, dtype=torch.long), target_token_ids=torch.tensor(targets, dtype=torch.long),
            cumulative_seq_lengths=torch.tensor([0, S], dtype=torch.int32), position_ids=torch.arange(0, S),
            loss_weights=torch.tensor(mask, dtype=torch.float32), input_images=images, input_image_locations=locations,
        )

    def collate(self, batch: List[TextImageDatasetItem]) -> TextDatasetBatch:
        return collate_items(batch)

    @staticmethod
    def sync_batch_to_model_parallel(topology: Optional[Topology], batch: Optional[TextDatasetBatch]) -> TextDatasetBatch:
        return sync_text_image_batch(topology, batch)


class TextImageBlendedDataset(BaseBlendedDataset[TextImageDataset]):
    pass
