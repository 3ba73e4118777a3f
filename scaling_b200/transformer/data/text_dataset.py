"""Pre-training text datasets: fixed-length windows packed from tokenised documents.

``TextDataset`` reads documents from a memory map (or retryable file reads), shuffles the document
order with ``numpy.random.RandomState(seed)`` and walks it emitting ``(document, start, end)`` pieces
until a window holds ``sequence_length + 1`` tokens; the last token of a window is the first of the
next (it is both target and next input), the unfilled tail is dropped, and ``only_full_sequences``
skips document remainders that cannot fill a fresh window except every n-th time.  The window index
is cached as a memory map next to the data (rank 0 builds, others wait) under the reference's file
names (src/scaling/transformer/data/text_dataset.py:26-469).  ``SyntheticTextDataset`` yields seeded
uniform-random token windows of the same shape for benchmarks and tests.
"""

from __future__ import annotations

import hashlib
import json
import time
from pathlib import Path
from typing import Optional, Union

import numpy as np
import torch
import torch.distributed as dist

from ...core.data.blended_dataset import BaseBlendedDataset
from ...core.data import BaseDataset, BaseDatasetItem, FileDataset, MemoryMapDataset, MemoryMapDatasetBuilder, broadcast_data
from ...parallel.topology import Topology
from .text_dataset_batch import TextDatasetBatch, TextDatasetBatchBeforeSync

POLL_SECONDS = 1.0


class TextDatasetItem(BaseDatasetItem):
    def __init__(self, token_ids: torch.Tensor):
        self.token_ids = token_ids


def pack_windows(doc_sizes, doc_order, sequence_length: int, only_full_sequences: bool = False,
                 allow_incomplete_sequences_every_n: int = 0) -> list[np.ndarray]:
    """Window index: one flat int64 array of ``(doc, start, end)`` triples per window of ``sequence_length + 1`` tokens."""
    want = sequence_length + 1
    windows: list[np.ndarray] = []
    pieces: list[tuple[int, int, int]] = []
    filled = 0
    full_count = partial_count = 0
    in_partial = False
    for doc in doc_order:
        size = int(doc_sizes[doc])
        pos = 0
        while pos < size - 1:  # the last token of a document can only serve as a target
            end = min(size, pos + want - filled)
            if only_full_sequences and not in_partial:
                if end - pos < want:
                    n = allow_incomplete_sequences_every_n
                    if n != 0 and (full_count / n) - partial_count >= 1:
                        in_partial = True
                    else:
                        break
                else:
                    full_count += 1
            filled += end - pos
            pieces.append((int(doc), pos, end))
            if filled == want:
                windows.append(np.asarray(pieces, dtype=np.int64).reshape(-1))
                pieces, filled = [], 0
                if in_partial:
                    partial_count += 1
                in_partial = False
            pos = end - 1
    return windows


class TextDataset(BaseDataset[TextDatasetItem, TextDatasetBatchBeforeSync, TextDatasetBatch]):
    def __init__(self, data_prefix: Path, sequence_length: int, seed: int, legacy_dataset: bool = False,
                 load_mmap_index_to_memory: bool = False, load_data_item_mmap_index_to_memory: bool = False,
                 only_full_sequences: bool = False, allow_incomplete_sequences_every_n: int = 0,
                 use_mmap: bool = True, shuffle: bool = True, reset_attention_mask: bool = True,
                 reset_position_ids: bool = True):
        self.use_mmap = use_mmap
        self.sequence_length = sequence_length
        self.legacy_dataset = legacy_dataset
        self.load_mmap_index_to_memory = load_mmap_index_to_memory
        self.load_data_item_mmap_index_to_memory = load_data_item_mmap_index_to_memory
        self.only_full_sequences = only_full_sequences
        self.allow_incomplete_sequences_every_n = allow_incomplete_sequences_every_n
        self.reset_attention_mask = reset_attention_mask
        self.reset_position_ids = reset_position_ids
        if legacy_dataset:
            from .legacy_dataset.indexed_dataset import make_dataset

            assert not (load_mmap_index_to_memory or load_data_item_mmap_index_to_memory or only_full_sequences), (
                "index-in-memory and full-sequence options are not available for legacy datasets"
            )
            self.memory_map = make_dataset(str(data_prefix))
        else:
            cls = MemoryMapDataset if use_mmap else FileDataset
            self.memory_map = cls(prefix_path=data_prefix, load_index_to_memory=load_mmap_index_to_memory)
        self.data_item_index: Union[MemoryMapDataset, FileDataset, None] = None
        super().__init__(seed=seed, shuffle=shuffle, data_prefix=data_prefix)

    def ident(self) -> str:
        return f"{hashlib.md5(str(self.data_prefix).encode('utf-8')).hexdigest()}-seq-{self.sequence_length}"

    def get_data_index_cache_filename_stem(self, seed: int) -> str:
        stem = str(self.data_prefix) + f"_index_cache_decoder_dataset_seed_{seed}_seq_len_{self.sequence_length}"
        if self.only_full_sequences:
            stem += f"_only_full_sequences_allow_incomplete_sequences_every_n_{self.allow_incomplete_sequences_every_n}"
        return stem

    def _doc_sizes(self) -> np.ndarray:
        sizes = self.memory_map.sizes
        return np.asarray(sizes() if callable(sizes) else sizes)

    def set_seed(self, seed: int, shuffle: bool = True) -> None:
        if self.seed is not None and self.seed == seed:
            return
        self.seed = seed
        stem = Path(self.get_data_index_cache_filename_stem(seed))
        meta = Path(str(stem) + ".meta.json")
        files = [Path(str(stem) + ext) for ext in (".bin", ".idx", ".meta.json")]
        builder_rank = (not dist.is_initialized()) or dist.get_rank() == 0
        if not meta.is_file() and builder_rank:
            for f in files[:2]:
                f.unlink(missing_ok=True)
            order = np.arange(len(self.memory_map))
            if shuffle:
                np.random.RandomState(seed=seed).shuffle(order)
            builder = MemoryMapDatasetBuilder(stem, dtype=np.dtype(np.int64), index_dtype=np.dtype(np.int64))
            for w in pack_windows(self._doc_sizes(), order, self.sequence_length, self.only_full_sequences,
                                  self.allow_incomplete_sequences_every_n):
                builder.add(w)
            builder.finalize()
        waited = 0.0
        while not all(f.is_file() for f in files):
            time.sleep(POLL_SECONDS)
            waited += POLL_SECONDS
            if waited % 60 < POLL_SECONDS:
                print(f"TextDataset waiting on index for seed {seed} for {Path(self.data_prefix).name}", flush=True)
        cls = MemoryMapDataset if self.use_mmap else FileDataset
        self.data_item_index = cls(prefix_path=stem, load_index_to_memory=self.load_data_item_mmap_index_to_memory)

    def __len__(self) -> int:
        return len(self.data_item_index)  # type: ignore[arg-type]

    def __getitem__(self, index: int) -> TextDatasetItem:
        assert self.data_item_index is not None, "data item index not set"
        triples = np.asarray(self.data_item_index[int(index)]).reshape(-1, 3)
        parts = [np.asarray(self.memory_map[int(d)][int(a):int(b)]) for d, a, b in triples]
        return TextDatasetItem(token_ids=torch.from_numpy(np.concatenate(parts).astype(np.int64)))

    def collate(self, batch: list[TextDatasetItem]) -> TextDatasetBatchBeforeSync:
        return TextDatasetBatchBeforeSync(
            token_ids=torch.stack([b.token_ids for b in batch]), reset_attention_mask=self.reset_attention_mask,
            reset_position_ids=self.reset_position_ids,
        )

    @staticmethod
    def sync_batch_to_model_parallel(topology: Optional[Topology],
                                     batch: Optional[TextDatasetBatchBeforeSync]) -> TextDatasetBatch:
        if topology is None:
            assert batch is not None
            ids, ram, rpi = batch.token_ids, batch.reset_attention_mask, batch.reset_position_ids
        else:
            if topology.model_parallel_rank == 0:
                assert batch is not None
                tensors = [batch.token_ids, torch.tensor([int(batch.reset_attention_mask)], dtype=torch.int64),
                           torch.tensor([int(batch.reset_position_ids)], dtype=torch.int64)]
                flags = (batch.reset_attention_mask, batch.reset_position_ids)
            else:
                assert batch is None
                tensors, flags = [None, None, None], None
            if topology.config.model_parallel_size == 1:
                ids = tensors[0].to(topology.device, non_blocking=True)  # flags are known locally: no host sync
                ram, rpi = flags  # type: ignore[misc]
            else:
                out = broadcast_data(tensors=tensors, dtype=torch.long, topology=topology)
                ids, ram, rpi = out[0], bool(out[1].item()), bool(out[2].item())
        return TextDatasetBatch(input_token_ids=ids[:, :-1], target_token_ids=ids[:, 1:].contiguous(),
                                reset_attention_mask=ram, reset_position_ids=rpi)

    @staticmethod
    def jsonl_to_memory_map(data_file_jsonl: Path, prefix_path_memory_map: Path, tokenizer=None) -> None:
        """Tokenise ``{"text": ...}`` lines into a memory map, one document (plus EOS) per line."""
        if tokenizer is None:
            from ..tokenizer import Tokenizer

            tokenizer = Tokenizer.default()
        builder = MemoryMapDatasetBuilder(prefix_path=Path(prefix_path_memory_map))
        with open(Path(data_file_jsonl), "r", encoding="UTF-8") as f:
            for line in f:
                ids = tokenizer.encode(json.loads(line)["text"]) + [tokenizer.eos_token_id]
                builder.add(np_array=np.array(ids))
        builder.finalize()


class SyntheticTextDataset(BaseDataset[TextDatasetItem, TextDatasetBatchBeforeSync, TextDatasetBatch]):
    """``n_samples`` windows of ``sequence_length + 1`` token ids drawn uniformly from ``[low, vocab_size)``.

    Every item is a pure function of ``(data_seed, index)``, so all ranks and resumed runs see the same data.
    With ``low = 1`` no end-of-document token (id 0) occurs and every window is a single document.
    """

    def __init__(self, n_samples: int, sequence_length: int, vocab_size: int, seed: int = 42, data_seed: int = 1234,
                 low: int = 0, shuffle: bool = True, reset_attention_mask: bool = True,
                 reset_position_ids: bool = True, materialize: bool = True):
        self.n_samples = n_samples
        self.sequence_length = sequence_length
        self.vocab_size = vocab_size
        self.data_seed = data_seed
        self.low = low
        self.reset_attention_mask = reset_attention_mask
        self.reset_position_ids = reset_position_ids
        self._table: Optional[torch.Tensor] = None
        if materialize:
            g = torch.Generator().manual_seed(data_seed)
            self._table = torch.randint(low, vocab_size, (n_samples, sequence_length + 1), generator=g, dtype=torch.int64)
        super().__init__(seed=seed, shuffle=shuffle)

    def ident(self) -> str:
        return f"synthetic-{self.n_samples}-seq-{self.sequence_length}-vocab-{self.vocab_size}"

    def set_seed(self, seed: int, shuffle: bool = True) -> None:
        self.seed = seed
        self.order = np.random.RandomState(seed).permutation(self.n_samples) if shuffle else np.arange(self.n_samples)

    def __len__(self) -> int:
        return self.n_samples

    def __getitem__(self, index: int) -> TextDatasetItem:
        j = int(self.order[index])
        if self._table is not None:
            return TextDatasetItem(self._table[j])
        g = torch.Generator().manual_seed(self.data_seed * 1_000_003 + j)
        return TextDatasetItem(torch.randint(self.low, self.vocab_size, (self.sequence_length + 1,), generator=g,
                                             dtype=torch.int64))

    def collate(self, batch: list[TextDatasetItem]) -> TextDatasetBatchBeforeSync:
        return TextDatasetBatchBeforeSync(
            token_ids=torch.stack([b.token_ids for b in batch]), reset_attention_mask=self.reset_attention_mask,
            reset_position_ids=self.reset_position_ids,
        )

    sync_batch_to_model_parallel = staticmethod(TextDataset.sync_batch_to_model_parallel)


class TextBlendedDataset(BaseBlendedDataset[TextDataset]):
    """Several ``TextDataset``s blended by weight (src/scaling/transformer/data/text_dataset.py:455-469)."""


def __getattr__(name: str):
    # kept importable from here; the class lives in legacy_blended_dataset (which imports this module)
    if name == "LegacyBlendedDataset":
        from .legacy_blended_dataset import LegacyBlendedDataset

        return LegacyBlendedDataset
    raise AttributeError(name)
