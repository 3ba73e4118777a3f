"""Blend of text corpora whose blend index is stored as a legacy ("mmap" indexed-dataset) file pair.

Runs that were started with the legacy data stack keep their blend index next to the data as
``index_cache_blended_dataset_seed_{s}_seq_len_{L}_prefix_{md5}_weights_{md5}.bin/.idx`` plus a ``.done`` marker;
this class reads and writes exactly those files (so a resumed run sees the sample order it was trained on) while
the interleaving itself comes from the native index builder (src/scaling/transformer/data/legacy_blended_dataset.py:22-283).

Differences to ``TextBlendedDataset``: file names and format of the cache, weights may also be given per data
prefix through ``ep_maximum_dict`` (a rate limit per dataset for examples-proportional mixing), no second shuffle
of the index.
"""

from __future__ import annotations

import hashlib
import os
import time
from pathlib import Path
from typing import Optional, Sequence

import numpy as np
import torch

from ...core.data.blended_dataset import (BaseBlendedDataset, build_blend_index, weights_by_num_docs,
                                          weights_examples_proportional)
from ...core.data.blended_dataset_config import BlendedDatasetConfig
from ...core.logging import logger
from .legacy_dataset.indexed_dataset import MMapIndexedDataset, write_fixed_width_items
from .text_dataset import TextDataset

POLL_SECONDS = 5.0


class LegacyBlendedDataset(BaseBlendedDataset[TextDataset]):
    def __init__(self, seed: int, config: BlendedDatasetConfig, datasets: Sequence[TextDataset], shuffle: bool = True,
                 ep_maximum_dict: Optional[dict[str, int]] = None):
        # rate limit per dataset (key: stem of its data prefix) for examples-proportional mixing; datasets without
        # an entry fall back to ``config.ep_maximum`` and, failing that, to their own size (no limit)
        self.ep_maximum_dict = ep_maximum_dict
        self.poll_seconds = POLL_SECONDS
        super().__init__(seed=seed, config=config, datasets=datasets)

    # ------------------------------------------------------------------ cache files
    def get_data_index_cache_filename_stem(self, seed: int) -> str:
        assert self.config.cache_directory is not None, "cache directory is needed"
        self.config.cache_directory.mkdir(exist_ok=True, parents=True)
        prefixes = "-".join(Path(d.data_prefix).name for d in self.datasets)
        weights = "-".join(str(round(w * 100) / 100) for w in self.weights.tolist())
        return str(self.config.cache_directory / (
            f"index_cache_blended_dataset_seed_{seed}_seq_len_{self.datasets[0].sequence_length}"
            f"_prefix_{hashlib.md5(prefixes.encode('utf-8')).hexdigest()}"
            f"_weights_{hashlib.md5(weights.encode('utf-8')).hexdigest()}"))

    def get_data_index_cache_filename_bin(self, seed: int) -> str:
        return self.get_data_index_cache_filename_stem(seed) + ".bin"

    def get_data_index_cache_filename_idx(self, seed: int) -> str:
        return self.get_data_index_cache_filename_stem(seed) + ".idx"

    def get_data_index_cache_filename_done(self, seed: int) -> str:
        return self.get_data_index_cache_filename_stem(seed) + ".done"

    # ------------------------------------------------------------------ weights
    def _rate_limits(self, counts: list[int]):
        if self.ep_maximum_dict is None:
            return self.config.ep_maximum
        limits = []
        for ds, n in zip(self.datasets, counts):
            stem = Path(ds.data_prefix).stem
            if stem in self.ep_maximum_dict:
                limits.append(self.ep_maximum_dict[stem])
            elif self.config.ep_maximum is not None:
                limits.append(self.config.ep_maximum)
            else:
                limits.append(n)
        return limits

    def _compute_weights(self, counts: list[int]) -> np.ndarray:
        c = self.config
        if not c.weight_by_num_documents:
            return super()._compute_weights(counts)
        if not c.weight_examples_proportional:
            return weights_by_num_docs(counts, c.weighted_sampler_alpha)
        assert self.ep_maximum_dict is not None or c.ep_maximum is not None, (
            "ep_maximum should be defined when using examples_proportional sampling")
        limits = self._rate_limits(counts)
        if isinstance(limits, list):
            # a limit per dataset: clip the sizes one by one, then mix without a further common limit
            clipped = [min(n, k) for n, k in zip(counts, limits)]
            unbiased = np.asarray(counts, dtype=np.float64) / float(sum(counts))
            rates = np.asarray(clipped, dtype=np.float64) / float(sum(clipped))
            if c.ep_temperature != 1.0:
                rates = rates ** (1.0 / c.ep_temperature)
                rates = rates / rates.sum()
            w = rates / unbiased
            return w / w.sum()
        return weights_examples_proportional(counts, c.ep_temperature, limits)

    # ------------------------------------------------------------------ index
    def set_seed(self, seed: int, shuffle: bool = True) -> None:
        assert shuffle, "Blended datasets should always be shuffled"
        if seed == self.seed:
            return
        self.seed = seed
        self.random_index = None
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
        files = [Path(stem + ext) for ext in (".bin", ".idx", ".done")]
        is_builder = not torch.distributed.is_initialized() or torch.distributed.get_rank() == 0
        if not files[2].is_file() and is_builder:
            start = time.time()
            scale = self.weights / self.weights.max()
            rnd = (lambda x: int(round(x))) if self.config.weight_examples_proportional else int
            targets = [max(1, rnd(p * n)) for n, p in zip(counts, scale)]
            scratch = f"{stem}.pairs.{os.getpid()}"
            n_pairs = build_blend_index(targets, scratch, until_all=False)
            pairs = np.fromfile(scratch + ".bin", dtype=np.int64).reshape(n_pairs, 2)
            write_fixed_width_items(stem + ".bin", stem + ".idx", pairs.astype(np.int32))
            for ext in (".bin", ".input.json", ".meta.json"):
                os.remove(scratch + ext)
            with open(files[2], "w") as f:  # written last: marks a complete index
                f.write("True")
            logger.info(f"{self.__class__.__name__}: blend index of {n_pairs} items for seed {seed} "
                        f"built in {time.time() - start:.2f}s")
        waited = 0
        while not all(f.is_file() for f in files):
            waited += 1
            if waited % 12 == 0:
                rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else None
                logger.info(f"LegacyBlendedDataset waiting on index for seed {seed} on rank {rank}; elapsed "
                            f"{waited * self.poll_seconds / 60:.1f} minutes; present: "
                            + ", ".join(f"{f.name}: {f.is_file()}" for f in files))
            time.sleep(self.poll_seconds)
        self.dataset_indices = MMapIndexedDataset(stem)
        self.size = len(self.dataset_indices)

    def __getitem__(self, index: int):
        if self.size < self.config.minimum_dataset_size:
            index %= self.size
        if self.num_datasets == 1:
            return self.datasets[0][index]
        dataset_index, item_index = self.dataset_indices[index].tolist()
        return self.datasets[dataset_index][item_index]
