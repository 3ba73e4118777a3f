"""Activation record passed between transformer layers, and its tuple form.

The tuple consists of the non-None fields followed by the list of their names, which is what
travels over pipeline boundaries and through activation checkpointing
(src/scaling/transformer/model/layers/base.py:12-123).
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from ....core.data import BaseLayerIO
from ....core.nn.parallel_module import BaseLayer
from ...data.inference_settings import InferenceSettings
from ...data.text_dataset_batch import _FieldRecord


class TransformerLayerIO(_FieldRecord, BaseLayerIO):
    @staticmethod
    def field_names() -> list[str]:
        return ["activations", "position_ids", "cumulative_seq_lengths", "cumulative_seq_lengths_padded",
                "loss_weights", "inference_settings", "embeddings", "embeddings_head", "attention_scores_manipulation"]

    def __init__(self, activations: torch.Tensor, position_ids: torch.Tensor,
                 cumulative_seq_lengths_padded: Optional[torch.Tensor] = None,
                 cumulative_seq_lengths: Optional[torch.Tensor] = None, loss_weights: Optional[torch.Tensor] = None,
                 inference_settings: Optional[InferenceSettings] = None, embeddings: Optional[torch.Tensor] = None,
                 embeddings_head: Optional[torch.Tensor] = None,
                 attention_scores_manipulation: Optional[torch.Tensor] = None) -> None:
        self.activations = activations
        self.position_ids = position_ids
        self.cumulative_seq_lengths = cumulative_seq_lengths
        self.cumulative_seq_lengths_padded = cumulative_seq_lengths_padded
        self.loss_weights = loss_weights
        self.inference_settings = inference_settings
        self.embeddings = embeddings
        self.embeddings_head = embeddings_head
        self.attention_scores_manipulation = attention_scores_manipulation

    def evolve(self, **changes: Any) -> "TransformerLayerIO":
        """Copy with some fields replaced."""
        fields = {n: getattr(self, n) for n in self.field_names()}
        fields.update(changes)
        out = TransformerLayerIO(**fields)
        out._doc_ranges = getattr(self, "_doc_ranges", None)
        return out

    def document_ranges(self) -> Optional[tuple[torch.Tensor, torch.Tensor]]:
        """Per-token ``(document start, document end)`` for the fused attention kernel, derived once per micro
        batch from the fixed-length padded cumulative lengths (fixed shapes, no host synchronisation)."""
        cached = getattr(self, "_doc_ranges", None)
        if cached is not None:
            return cached
        padded = self.cumulative_seq_lengths_padded
        if padded is None or not padded.is_cuda or self.inference_settings is not None:
            return None
        from ...data.utils import document_ranges_from_padded

        # all tokens of the micro batch: under sequence parallelism the activations hold only this rank's share,
        # while attention runs on the gathered sequence
        if self.position_ids is not None:
            total = self.position_ids.numel()
        else:
            total = self.activations.shape[0] * self.activations.shape[1]
        self._doc_ranges = document_ranges_from_padded(padded, total)
        return self._doc_ranges


class TransformerLayerBaseIO(BaseLayer[TransformerLayerIO, TransformerLayerIO, TransformerLayerIO]):
    @staticmethod
    def input_to_tuple(input: TransformerLayerIO) -> tuple[Any, ...]:
        return input.as_tuple()

    @staticmethod
    def tuple_to_input(d: tuple[Any, ...]) -> TransformerLayerIO:
        return TransformerLayerIO.from_tuple(d)

    @staticmethod
    def output_to_tuple(output: TransformerLayerIO) -> tuple[Any, ...]:
        return output.as_tuple()

    @staticmethod
    def tuple_to_last_stage_activation(d: tuple[Any, ...]) -> TransformerLayerIO:
        return TransformerLayerIO.from_tuple(d)


def record_embedding(x: TransformerLayerIO, slot_layer_index: int, activations: torch.Tensor) -> None:
    """Store ``activations`` in the hidden-state buffer if this layer's output was requested."""
    s = x.inference_settings
    if s is not None and slot_layer_index in s.embedding_layers:
        assert x.embeddings is not None
        x.embeddings[s.embedding_layers.index(slot_layer_index)] = activations
