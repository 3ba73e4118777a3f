"""Blending of several datasets into one (src/scaling/core/data/blended_dataset.py:24-398).

Weights come from document counts (``p ** alpha`` re-normalised), from examples-proportional mixing with a rate
limit and a temperature, or from the configuration.  The blend itself is an index of (dataset, item) pairs in which
the sources are interleaved as evenly as their weights allow; it is built once per seed by the native builder
(``csrc/blend_index.cpp``) into ``cache_directory``, by global rank 0, and memory-mapped by every rank.
"""

from __future__ import annotations

import ctypes
import hashlib
import json
import os
import time
from pathlib import Path
from typing import Any, Generic, List, Optional, Sequence, TypeVar

import numpy as np
import torch

from ...parallel.topology import Topology
from ..logging import logger
from .base_dataset import BaseDataset, BaseDatasetBatch, BaseDatasetItem
from .blended_dataset_config import BlendedDatasetConfig

TDataset = TypeVar("TDataset", bound=BaseDataset)
TItem = TypeVar("TItem", bound=BaseDatasetItem)
TBatchBeforeSync = TypeVar("TBatchBeforeSync", bound=BaseDatasetBatch)
TBatch = TypeVar("TBatch", bound=BaseDatasetBatch)


def weights_by_num_docs(examples: Sequence[int], alpha: float = 0.3) -> np.ndarray:
    """Per-dataset multipliers ``q_i / p_i`` (normalised) with ``p_i`` the size share and ``q_i ∝ p_i ** alpha``.

    ``alpha`` < 1 boosts small datasets (XLM sampling, arXiv 1901.07291); multiplied by the document counts the
    weights give the number of items to take from each dataset.
    """
    n = np.asarray(examples, dtype=np.float64)
    p = n / n.sum()
    q = p ** alpha
    q = q / q.sum()
    # multiply by the reciprocal (not: divide): the item counts are int(weight * documents), and the last bit of the
    # weight decides whether a dataset contributes n or n - 1 items; this is the rounding of
    # src/scaling/core/data/blended_dataset.py:50-56, so the same corpora give the same blend
    w = q * (1 / p)
    return w / w.sum()


def weights_examples_proportional(examples: Sequence[int], temperature: float = 1.0,
                                  maximum: Optional[float] = None) -> np.ndarray:
    """Examples-proportional mixing (T5, arXiv 1910.10683 p. 31): rates ``min(e_m, K) / sum_n min(e_n, K)``,
    optionally raised to ``1 / T``; returned as multipliers on the document counts like ``weights_by_num_docs``."""
    assert temperature is not None and temperature != 0, "temperature is 0, expect non-zero temperature"
    n = np.asarray(examples, dtype=np.float64)
    p = n / n.sum()
    limited = n.copy()
    if maximum:
        assert maximum > 0, f"examples-proportional sampling requires maximum limit > 0 (current max = {maximum})"
        limited = np.minimum(limited, maximum)
    r = limited / limited.sum()
    if temperature != 1.0:
        r = r ** (1.0 / temperature)
        r = r / r.sum()
    w = r * (1 / p)  # reciprocal, as above
    return w / w.sum()


def build_blend_index(targets: Sequence[int], stem: str, until_all: bool = True) -> int:
    """Write ``{stem}.bin`` (int64 pairs), ``{stem}.input.json`` and ``{stem}.meta.json``; returns the pair count.
    ``until_all``: go on until every dataset has given its target number of items (datasets that are done drop out);
    ``False``: stop when the first dataset is done, as the legacy blend does."""
    from ...ops import _build

    arr = np.ascontiguousarray(np.asarray(targets, dtype=np.int64))
    lib_path = _build.LIB_PATH
    if not lib_path.exists():
        _build.build()
    lib = ctypes.CDLL(str(lib_path))
    fn = lib.sb200_blend_index_ex
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int]
    fn.restype = ctypes.c_long
    tmp = f"{stem}.bin.tmp.{os.getpid()}"
    count = int(fn(arr.ctypes.data, int(arr.size), tmp.encode(), int(until_all)))
    if count < 0:
        raise RuntimeError(f"blend index builder failed with code {count} for {stem}")
    os.replace(tmp, f"{stem}.bin")
    with open(f"{stem}.input.json", "w", encoding="UTF-8") as f:
        json.dump({"number_to_sample_by_dataset": arr.tolist()}, f)
    meta_tmp = f"{stem}.meta.json.tmp.{os.getpid()}"
    with open(meta_tmp, "w", encoding="UTF-8") as f:
        json.dump({"dtype": "int64", "shape": [count, 2]}, f)
    os.replace(meta_tmp, f"{stem}.meta.json")  # written last: its presence marks a complete index
    return count


class BaseBlendedDataset(BaseDataset, Generic[TItem, TBatchBeforeSync, TBatch, TDataset]):
    """Indexable union of ``datasets``; a single dataset passes through untouched.

    Generic over (item, batch before the tensor-parallel sync, batch, blended dataset class) like
    src/scaling/core/data/blended_dataset.py:128-135; ``BaseBlendedDataset[SomeDataset]`` names the last one alone."""

    def __class_getitem__(cls, params):  # type: ignore[no-untyped-def]
        if not isinstance(params, tuple):
            params = (BaseDatasetItem, BaseDatasetBatch, BaseDatasetBatch, params)
        return super().__class_getitem__(params)

    def __init__(self, seed: int, config: BlendedDatasetConfig, datasets: Sequence[TDataset]) -> None:
        self.config = config
        self.datasets: Sequence[TDataset] = datasets
        self.num_datasets = len(datasets)
        assert self.num_datasets > 0, "no datasets to blend"
        self.weights: np.ndarray = np.ones(self.num_datasets, dtype=np.float64) / self.num_datasets
        self.random_index: Optional[np.ndarray] = None
        self.dataset_indices: Any = None
        self.size = 0
        self.seed: Optional[int] = None
        self.set_seed(seed=seed, shuffle=True)

    # ------------------------------------------------------------------ identity / cache files
    def ident(self) -> str:
        prefix = hashlib.md5("-".join(d.ident() for d in self.datasets).encode("utf-8")).hexdigest()
        weights = hashlib.md5("-".join(str(round(w * 100) / 100) for w in self.weights.tolist()).encode("utf-8")).hexdigest()
        return f"{self.datasets[0].__class__.__name__}_prefix_{prefix}_weights_{weights}"

    def get_data_index_cache_filename_stem(self, seed: int) -> str:
        assert self.config.cache_directory is not None, "cache directory is needed"
        self.config.cache_directory.mkdir(exist_ok=True, parents=True)
        return str(self.config.cache_directory / f"index_cache_blended_dataset_seed_{seed}_{self.ident()}")

    def get_data_index_cache_filename_meta(self, seed: int) -> str:
        return self.get_data_index_cache_filename_stem(seed) + ".meta.json"

    def get_data_index_cache_filename_input(self, seed: int) -> str:
        return self.get_data_index_cache_filename_stem(seed) + ".input.json"

    def get_data_index_cache_filename_bin(self, seed: int) -> str:
        return self.get_data_index_cache_filename_stem(seed) + ".bin"

    # ------------------------------------------------------------------ dataset protocol
    def __len__(self) -> int:
        return max(self.size, self.config.minimum_dataset_size)

    def __getitem__(self, index: int):
        if self.size < self.config.minimum_dataset_size:
            index %= self.size
        if self.num_datasets == 1:
            return self.datasets[0][index]
        if self.random_index is not None:
            index = int(self.random_index[index])
        dataset_index, item_index = self.dataset_indices[index]
        return self.datasets[int(dataset_index)][int(item_index)]

    def _compute_weights(self, counts: list[int]) -> np.ndarray:
        c = self.config
        if c.weight_by_num_documents:
            if c.weight_examples_proportional:
                return weights_examples_proportional(counts, c.ep_temperature, c.ep_maximum)
            return weights_by_num_docs(counts, c.weighted_sampler_alpha)
        assert c.weights is not None and len(c.weights) == len(self.datasets)
        w = np.asarray(c.weights, dtype=np.float64)
        assert w.sum() > 0.0
        return w / w.sum()

    def set_seed(self, seed: int, shuffle: bool = True) -> None:
        if seed == self.seed:
            return
        self.seed = seed
        assert shuffle, "Blended datasets should always be shuffled"
        if self.num_datasets == 1:
            self.datasets[0].set_seed(seed=seed, shuffle=shuffle)
            self.size = len(self.datasets[0])
            return
        counts = []
        for ds in self.datasets:
            ds.set_seed(seed=seed, shuffle=shuffle)
            counts.append(len(ds))
        self.weights = self._compute_weights(counts)

        stem = self.get_data_index_cache_filename_stem(seed)
        meta_file = Path(self.get_data_index_cache_filename_meta(seed))
        bin_file = Path(self.get_data_index_cache_filename_bin(seed))
        input_file = Path(self.get_data_index_cache_filename_input(seed))
        is_builder = not torch.distributed.is_initialized() or torch.distributed.get_rank() == 0
        if not meta_file.is_file() and is_builder:
            start = time.time()
            scale = self.weights / self.weights.max()
            rnd = (lambda x: int(round(x))) if self.config.weight_examples_proportional else int
            targets = [max(1, rnd(p * n)) for n, p in zip(counts, scale)]
            n_pairs = build_blend_index(targets, stem)
            logger.info(f"{self.__class__.__name__}: blend index of {n_pairs} items for seed {seed} "
                        f"built in {time.time() - start:.2f}s")
        waited = 0
        while not (bin_file.is_file() and input_file.is_file() and meta_file.is_file()):
            waited += 1
            if waited % 12 == 0:
                logger.info(f"BlendedDataset waiting on index for seed {seed}; elapsed {waited * 5 / 60:.1f} minutes")
            time.sleep(5)
        with open(meta_file, "r", encoding="UTF-8") as f:
            self.dataset_meta = json.load(f)
        dtype, shape = np.dtype(self.dataset_meta["dtype"]), tuple(self.dataset_meta["shape"])
        if self.config.load_dataset_indices_to_memory:
            self.dataset_indices = np.fromfile(bin_file, dtype=dtype).reshape(shape)
        else:
            self.dataset_indices = np.memmap(bin_file, mode="r", order="C", dtype=dtype, shape=shape)
        self.size = shape[0]
        # optional second shuffle so that neighbouring items do not follow the deterministic interleaving
        # (an index held in memory is shuffled in place; a memory-mapped one is read through `random_index`, which is
        # the identity without the shuffle)
        reshuffle = self.config.shuffle_dataset_indices and shuffle
        rng = np.random.RandomState(seed=seed)
        if self.config.load_dataset_indices_to_memory:
            self.random_index = None
            if reshuffle:
                rng.shuffle(self.dataset_indices)
        else:
            self.random_index = np.arange(self.size)
            if reshuffle:
                rng.shuffle(self.random_index)

    def collate(self, batch: List[Any]):
        return self.datasets[0].collate(batch=batch)

    @staticmethod
    def sync_batch_to_model_parallel(topology: Topology, batch: Any):
        raise NotImplementedError("use the sync function of the blended datasets' own class")

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}_{self.datasets[0].__class__.__name__}"
