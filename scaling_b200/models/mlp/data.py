"""Datasets of the MLP application: seeded synthetic classification data, or MNIST idx files."""

from __future__ import annotations

import gzip
import struct
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from ...core.data import BaseDataset, BaseDatasetBatch, BaseDatasetItem, broadcast_data
from ...parallel.topology import Topology


class MLPDatasetItem(BaseDatasetItem):
    def __init__(self, input: torch.Tensor, target: torch.Tensor):
        self.input = input
        self.target = target


class MLPDatasetBatch(BaseDatasetBatch):
    def __init__(self, inputs: Optional[torch.Tensor] = None, targets: Optional[torch.Tensor] = None):
        self.inputs = inputs
        self.targets = targets

    def only_inputs(self) -> "MLPDatasetBatch":
        return MLPDatasetBatch(inputs=self.inputs)

    def only_targets(self) -> "MLPDatasetBatch":
        return MLPDatasetBatch(targets=self.targets)


class _ClassificationDataset(BaseDataset[MLPDatasetItem, MLPDatasetBatch, MLPDatasetBatch]):
    inputs: torch.Tensor
    targets: torch.Tensor

    def __len__(self) -> int:
        return self.inputs.shape[0]

    def __getitem__(self, index: int) -> MLPDatasetItem:
        j = int(self.order[index])
        return MLPDatasetItem(self.inputs[j], self.targets[j])

    def set_seed(self, seed: int, shuffle: bool = True) -> None:
        self.seed = seed
        n = self.inputs.shape[0] if hasattr(self, "inputs") else 0
        self.order = np.random.RandomState(seed).permutation(n) if shuffle else np.arange(n)

    def collate(self, batch: list[MLPDatasetItem]) -> MLPDatasetBatch:
        return MLPDatasetBatch(inputs=torch.stack([b.input for b in batch]),
                               targets=torch.stack([b.target for b in batch]))

    @staticmethod
    def sync_batch_to_model_parallel(topology: Topology, batch: Optional[MLPDatasetBatch]) -> MLPDatasetBatch:
        if topology.model_parallel_rank == 0:
            assert batch is not None
            floats, ints = [batch.inputs], [batch.targets]
        else:
            floats, ints = [None], [None]
        inputs = broadcast_data(floats, torch.float32, topology)[0]
        targets = broadcast_data(ints, torch.int64, topology)[0]
        return MLPDatasetBatch(inputs=inputs, targets=targets)


class SyntheticClassificationDataset(_ClassificationDataset):
    """Inputs uniform in [0, 1), labels uniform in [0, classes) - fixed by ``data_seed``."""

    def __init__(self, n_samples: int = 4096, input_dim: int = 784, classes: int = 10, data_seed: int = 0,
                 seed: int = 42, shuffle: bool = True):
        g = torch.Generator().manual_seed(data_seed)
        self.inputs = torch.rand(n_samples, input_dim, generator=g)
        self.targets = torch.randint(0, classes, (n_samples,), generator=g)
        super().__init__(seed=seed, shuffle=shuffle)

    def ident(self) -> str:
        return f"synthetic_classification_{self.inputs.shape[0]}"


def _read_idx(path: Path) -> np.ndarray:
    opener = gzip.open if path.suffix == ".gz" else open
    with opener(path, "rb") as f:
        _, _, dims = struct.unpack(">HBB", f.read(4))
        shape = tuple(struct.unpack(">I", f.read(4))[0] for _ in range(dims))
        return np.frombuffer(f.read(), dtype=np.uint8).reshape(shape)


class MNISTDataset(_ClassificationDataset):
    """MNIST from the original idx files in ``root`` (``train-images-idx3-ubyte[.gz]`` ...)."""

    def __init__(self, root: Path, train: bool = True, seed: int = 42, shuffle: bool = True):
        prefix = "train" if train else "t10k"
        root = Path(root)

        def find(stem: str) -> Path:
            for cand in (root / stem, root / (stem + ".gz")):
                if cand.is_file():
                    return cand
            raise FileNotFoundError(f"{stem}[.gz] not found in {root}")

        images = _read_idx(find(f"{prefix}-images-idx3-ubyte")).astype(np.float32) / 255.0
        labels = _read_idx(find(f"{prefix}-labels-idx1-ubyte")).astype(np.int64)
        self.inputs = torch.from_numpy((images - 0.1307) / 0.3081).reshape(images.shape[0], -1)
        self.targets = torch.from_numpy(labels)
        super().__init__(seed=seed, shuffle=shuffle)

    def ident(self) -> str:
        return "mnist"
