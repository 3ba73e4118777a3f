"""Datasets of the MLP example (step 3 of the walk-through): items, batches, a synthetic task and MNIST."""

from scaling_b200.models.mlp.data import MLPDatasetBatch, MLPDatasetItem, MNISTDataset, SyntheticClassificationDataset

__all__ = ["MLPDatasetBatch", "MLPDatasetItem", "MNISTDataset", "SyntheticClassificationDataset"]
