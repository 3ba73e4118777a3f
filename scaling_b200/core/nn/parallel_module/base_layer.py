"""Contract between the pipeline engine and a layer.

The engine moves activations between stages and through activation checkpointing as flat tuples;
a layer states how its typed input / output records map to such tuples
(reference: src/scaling/core/nn/parallel_module/base_layer.py:16-70).
"""

from __future__ import annotations

from abc import abstractmethod
from typing import Any, Generic, TypeVar

import torch

from ...data.base_layer_io import BaseLayerIO

BaseLossInputGeneric = TypeVar("BaseLossInputGeneric")
BaseLossOutputGeneric = TypeVar("BaseLossOutputGeneric", torch.Tensor, tuple)
BaseDatasetBatchGeneric = TypeVar("BaseDatasetBatchGeneric")
BaseLayerInputGeneric = TypeVar("BaseLayerInputGeneric")
BaseLayerOutputGeneric = TypeVar("BaseLayerOutputGeneric", bound=BaseLayerIO)
BaseLayerLastLayerOutputGeneric = TypeVar("BaseLayerLastLayerOutputGeneric", bound=BaseLayerIO)


class BaseLayer(torch.nn.Module, Generic[BaseLayerInputGeneric, BaseLayerOutputGeneric, BaseLayerLastLayerOutputGeneric]):
    @abstractmethod
    def forward(self, x: BaseLayerInputGeneric) -> BaseLayerOutputGeneric:
        raise NotImplementedError

    @staticmethod
    @abstractmethod
    def input_to_tuple(input: BaseLayerInputGeneric) -> tuple[Any, ...]:
        """Flatten the layer input for pipe communication / activation checkpointing."""
        raise NotImplementedError

    @staticmethod
    @abstractmethod
    def tuple_to_input(d: tuple[Any, ...]) -> BaseLayerInputGeneric:
        """Inverse of ``input_to_tuple``."""
        raise NotImplementedError

    @staticmethod
    @abstractmethod
    def output_to_tuple(output: BaseLayerOutputGeneric) -> tuple[Any, ...]:
        """Flatten the layer output for pipe communication / activation checkpointing."""
        raise NotImplementedError

    @staticmethod
    @abstractmethod
    def tuple_to_last_stage_activation(d: tuple[Any, ...]) -> BaseLayerLastLayerOutputGeneric:
        """Rebuild the record handed to the loss function from the last layer's tuple."""
        raise NotImplementedError

    def _forward_tuple_input(self, *args: Any) -> Any:
        return self(self.tuple_to_input(tuple(args)))
