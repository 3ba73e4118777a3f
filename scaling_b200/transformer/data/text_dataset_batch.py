"""Batch records of the text datasets (src/scaling/transformer/data/text_dataset_batch.py:16-149)."""

from __future__ import annotations

from typing import Any, Optional

import torch

from ...core.data import BaseDatasetBatch
from .inference_settings import InferenceSettings
from .utils import (
    add_cumulative_seq_lengths_padding,
    get_cumulative_seq_lengths,
    get_cumulative_seq_lengths_padded,
    get_position_ids,
    remove_cumulative_seq_lengths_padding,
)


def _capturing() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


class _FieldRecord:
    """Mixin: (de)serialise the non-None fields as a flat tuple whose last entry lists the field names."""

    @staticmethod
    def field_names() -> list[str]:
        raise NotImplementedError

    def as_tuple(self) -> tuple[Any, ...]:
        names = [n for n in self.field_names() if getattr(self, n) is not None]
        return tuple([getattr(self, n) for n in names] + [names])

    @classmethod
    def from_tuple(cls, d: tuple[Any, ...]):
        names, values = d[-1], d[:-1]
        assert len(names) == len(values)
        return cls(**dict(zip(names, values)))


class TextDatasetBatchBeforeSync(BaseDatasetBatch):
    def __init__(self, token_ids: torch.Tensor, reset_attention_mask: bool = True, reset_position_ids: bool = True):
        self.token_ids = token_ids
        self.reset_attention_mask = reset_attention_mask
        self.reset_position_ids = reset_position_ids


class TextDatasetBatch(_FieldRecord, BaseDatasetBatch):
    @staticmethod
    def field_names() -> list[str]:
        return ["input_token_ids", "input_images", "input_image_locations", "target_token_ids", "position_ids",
                "cumulative_seq_lengths", "cumulative_seq_lengths_padded", "loss_weights", "inference_settings",
                "embeddings"]

    def __init__(self, input_token_ids: Optional[torch.Tensor] = None, input_images: Optional[torch.Tensor] = None,
                 input_image_locations: Optional[torch.Tensor] = None, target_token_ids: Optional[torch.Tensor] = None,
                 position_ids: Optional[torch.Tensor] = None, cumulative_seq_lengths: Optional[torch.Tensor] = None,
                 cumulative_seq_lengths_padded: Optional[torch.Tensor] = None,
                 loss_weights: Optional[torch.Tensor] = None, inference_settings: Optional[InferenceSettings] = None,
                 embeddings: Optional[torch.Tensor] = None, reset_attention_mask: bool = True,
                 reset_position_ids: bool = True) -> None:
        self.input_token_ids = input_token_ids
        self.input_images = input_images
        self.input_image_locations = input_image_locations
        self.target_token_ids = target_token_ids
        self.position_ids = position_ids
        self.cumulative_seq_lengths = cumulative_seq_lengths
        self.cumulative_seq_lengths_padded = cumulative_seq_lengths_padded
        self.loss_weights = loss_weights
        self.inference_settings = inference_settings
        self.embeddings = embeddings
        if input_token_ids is None:
            return
        if self.cumulative_seq_lengths_padded is None:
            if self.cumulative_seq_lengths is not None:
                b, s = input_token_ids.shape
                self.cumulative_seq_lengths_padded = add_cumulative_seq_lengths_padding(self.cumulative_seq_lengths, b * (s + 1))
            else:
                self.cumulative_seq_lengths_padded = get_cumulative_seq_lengths_padded(input_token_ids, reset_attention_mask)
        # the un-padded form has a data-dependent length; while a CUDA graph is being captured only the padded
        # form exists and consumers derive what they need from it
        if self.cumulative_seq_lengths is None and not _capturing():
            self.cumulative_seq_lengths = remove_cumulative_seq_lengths_padding(self.cumulative_seq_lengths_padded)
        if self.position_ids is None:
            self.position_ids = get_position_ids(input_token_ids, reset_position_ids)
        if self.loss_weights is None:
            self.loss_weights = torch.ones_like(input_token_ids, dtype=torch.float).contiguous()

    def only_inputs(self) -> "TextDatasetBatch":
        return TextDatasetBatch(
            input_token_ids=self.input_token_ids, input_images=self.input_images,
            input_image_locations=self.input_image_locations, position_ids=self.position_ids,
            cumulative_seq_lengths=self.cumulative_seq_lengths, loss_weights=self.loss_weights,
        )

    def only_targets(self) -> "TextDatasetBatch":
        return TextDatasetBatch(target_token_ids=self.target_token_ids, loss_weights=self.loss_weights)
