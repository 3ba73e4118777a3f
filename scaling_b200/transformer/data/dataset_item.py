"""Item record of the prompt / completion and text-image datasets (src/scaling/transformer/data/dataset_item.py:6-32)."""

from __future__ import annotations

from typing import Optional

import torch

from ...core.data import BaseDatasetItem


class TextImageDatasetItem(BaseDatasetItem):
    """One fixed-length sequence: tokens, targets, loss weights and, optionally, the images spliced into the prompt
    (``input_image_locations``: (start, end) token ranges that the image encoder's outputs replace)."""

    def __init__(self, input_token_ids: torch.Tensor, target_token_ids: torch.Tensor,
                 cumulative_seq_lengths: torch.Tensor, position_ids: torch.Tensor, loss_weights: torch.Tensor,
                 input_images: Optional[list[torch.Tensor]] = None,
                 input_image_locations: Optional[list[tuple[int, int]]] = None) -> None:
        self.input_token_ids = input_token_ids
        self.target_token_ids = target_token_ids
        self.cumulative_seq_lengths = cumulative_seq_lengths
        self.position_ids = position_ids
        self.loss_weights = loss_weights
        self.input_images = input_images
        self.input_image_locations = input_image_locations
