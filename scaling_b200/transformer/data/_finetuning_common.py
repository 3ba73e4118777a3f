"""Pieces shared by the prompt / completion, chat and text-image datasets: batching of ``TextImageDatasetItem``s and
the tensor-parallel broadcast of such batches (the collate / sync halves of
src/scaling/transformer/data/finetuning_text_dataset.py:249-357 and finetuning_chat_dataset.py:230-342)."""

from __future__ import annotations

from typing import Any, Callable, Optional

import torch

from ...core.data import broadcast_data
from ...parallel.topology import Topology
from .dataset_item import TextImageDatasetItem
from .text_dataset_batch import TextDatasetBatch
from .utils import get_cumulative_seq_lengths

IMAGE_ENCODER_TOKEN_COUNTS = 144   # tokens one encoded image occupies in the prompt
IMAGE_SIZE = (384, 384)

_TRANSFORM: Optional[Callable[[Any], torch.Tensor]] = None


def image_transform() -> Callable[[Any], torch.Tensor]:
    """PIL image -> normalised ``[3, 384, 384]`` tensor (created on first use: pulls in the image stack)."""
    global _TRANSFORM
    if _TRANSFORM is None:
        from ..model.image_encoder import clip_transform

        _TRANSFORM = clip_transform(IMAGE_SIZE)
    return _TRANSFORM


def shift_locations(locations: Optional[list[tuple[int, int]]], by: int) -> Optional[list[tuple[int, int]]]:
    if locations is None or by == 0:
        return locations
    return [(a + by, b + by) for a, b in locations]


def collate_items(batch: list[TextImageDatasetItem]) -> TextDatasetBatch:
    """Stack fixed-length items; images of all rows are concatenated, with ``[row, start, end]`` per image.  Tensors
    stay on the host: the loader runs in worker processes."""
    ids = torch.stack([b.input_token_ids for b in batch])
    images = locations = None
    if any(b.input_images for b in batch):
        imgs, locs = [], []
        for row, b in enumerate(batch):
            row_images = b.input_images or []
            row_locations = b.input_image_locations or []
            assert len(row_images) == len(row_locations)
            for img, (start, end) in zip(row_images, row_locations):
                imgs.append(img)
                locs.append([row, start, end])
        images = torch.stack(imgs, dim=0)
        locations = torch.tensor(locs, dtype=torch.long)
    return TextDatasetBatch(
        input_token_ids=ids,
        target_token_ids=torch.stack([b.target_token_ids for b in batch]),
        cumulative_seq_lengths=get_cumulative_seq_lengths(ids, reset_attention_mask=False),
        position_ids=torch.stack([b.position_ids for b in batch]),
        loss_weights=torch.stack([b.loss_weights for b in batch]),
        input_images=images, input_image_locations=locations,
    )


def sync_text_image_batch(topology: Optional[Topology], batch: Optional[TextDatasetBatch]) -> TextDatasetBatch:
    """Tensor-parallel rank 0 holds the batch; the others receive it.  Absent images travel as a ``-1`` marker."""
    if topology is None:
        assert batch is not None
        return batch
    if topology.model_parallel_rank == 0:
        assert batch is not None
        batch.contiguous_()
        assert batch.cumulative_seq_lengths_padded is not None
        longs: list[Optional[torch.Tensor]] = [
            batch.input_token_ids, batch.target_token_ids, batch.cumulative_seq_lengths_padded.to(torch.long),
            batch.position_ids,
            batch.input_image_locations if batch.input_image_locations is not None else torch.tensor([-1]),
        ]
        floats: list[Optional[torch.Tensor]] = [
            batch.loss_weights, batch.input_images if batch.input_images is not None else torch.tensor([-1.0]),
        ]
    else:
        assert batch is None
        longs, floats = [None] * 5, [None] * 2
    lt = broadcast_data(tensors=longs, dtype=torch.long, topology=topology)
    ft = broadcast_data(tensors=floats, dtype=torch.float32, topology=topology)
    no_images = bool((lt[4] == -1).all())
    return TextDatasetBatch(
        input_token_ids=lt[0], target_token_ids=lt[1], cumulative_seq_lengths_padded=lt[2].to(torch.int32),
        position_ids=lt[3], loss_weights=ft[0], input_images=None if no_images else ft[1],
        input_image_locations=None if no_images else lt[4],
    )
