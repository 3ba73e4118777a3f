"""Resumable, data-parallel aware batch sampler and an endless data loader.

Sampling rule (src/scaling/core/data/dataloader.py:38-94): with ``usable = (len // micro // dp) *
micro * dp`` samples per epoch, the epoch is ``consumed // usable`` and the dataset is re-seeded with
``seed + epoch``; data-parallel rank ``r`` draws indices ``i * dp + r + consumed_in_epoch`` and chunks
them into micro batches; every yielded micro batch advances ``consumed`` by ``micro * dp``.  Resuming
is constructing the loader with the ``consumed_samples`` stored in the context.
"""

from __future__ import annotations

from typing import Any, Iterator, Optional

import torch

from ...parallel.topology import Topology
from ..logging import logger
from .base_dataset import BaseDataset


class RandomSampler:
    def __init__(self, dataset: BaseDataset, seed: int, consumed_samples: int, topology: Topology,
                 shuffle: bool = True) -> None:
        self.dataset = dataset
        self.seed = seed
        self.consumed_samples = consumed_samples
        self.topology = topology
        self.shuffle = shuffle
        micro, dp = topology.config.micro_batch_size, topology.config.data_parallel_size
        self.total_samples = len(dataset)
        self.total_micro_batches = self.total_samples // micro
        self.total_micro_batches_per_data_parallel = self.total_micro_batches // dp
        self.usable_total_samples = self.total_micro_batches_per_data_parallel * micro * dp
        assert self.usable_total_samples > 0, (
            "not usable samples; this means that the dataset is too small for the provided data parallel size "
            "and micro batch size"
        )

    def __len__(self) -> int:
        return self.total_micro_batches

    def __iter__(self) -> Iterator[list[int]]:
        micro, dp = self.topology.config.micro_batch_size, self.topology.config.data_parallel_size
        epoch, done = divmod(self.consumed_samples, self.usable_total_samples)
        remaining = self.usable_total_samples - done
        logger.debug(f"dataset epoch {epoch}: {done} of {self.usable_total_samples} usable samples consumed")
        self.dataset.set_seed(seed=self.seed + epoch, shuffle=self.shuffle)
        first = self.topology.data_parallel_rank + done
        indices = [first + i * dp for i in range(remaining // dp)]
        assert len(indices) % micro == 0, "dataset index count is not a multiple of micro batch size"
        for start in range(0, len(indices), micro):
            self.consumed_samples += micro * dp
            yield indices[start:start + micro]


class DataLoader:
    """Endless iterator over micro batches of this data-parallel rank."""

    def __init__(self, seed: int, consumed_samples: int, dataset: BaseDataset, topology: Topology,
                 num_workers: int = 0, pin_memory: bool = True, prefetch_factor: Optional[int] = None,
                 shuffle: bool = True) -> None:
        self.seed = seed
        self.consumed_samples = consumed_samples
        self.dataset = dataset
        self.topology = topology
        assert len(dataset) >= topology.config.micro_batch_size, (
            f"cannot instantiate data loader with micro_batch_size {topology.config.micro_batch_size} "
            f"because dataset has only length {len(dataset)}"
        )
        self.sampler = RandomSampler(dataset, seed, consumed_samples, topology, shuffle)
        # torch's loader draws a base seed whenever an iterator is created (at the first batch, and again at every
        # new epoch): from a generator of its own, so that the global stream, which dropout reads, is the same
        # whether a run started here or was resumed here
        self._loader_generator = torch.Generator()
        self._loader_generator.manual_seed(seed)
        self.dataloader = torch.utils.data.DataLoader(
            dataset=dataset, batch_sampler=self.sampler, num_workers=num_workers, collate_fn=dataset.collate,
            pin_memory=pin_memory and torch.cuda.is_available(), prefetch_factor=prefetch_factor,
            generator=self._loader_generator,
        )
        self.iterator = self._iterate()

    def _iterate(self) -> Iterator[Any]:
        while True:
            yield from self.dataloader

    def __iter__(self) -> "DataLoader":
        return self

    def __next__(self) -> Any:
        return next(self.iterator)
