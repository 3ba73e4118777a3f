"""Activation functions selectable by config (src/scaling/core/nn/activation_function.py:7-17)."""

from enum import Enum
from typing import Callable

import torch

from ...ops import functional as K


class ActivationFunction(Enum):
    GELU = "gelu"
    SILU = "silu"


def get_activation_function(activation_function: ActivationFunction) -> Callable[..., torch.Tensor]:
    if activation_function == ActivationFunction.GELU:
        return K.gelu
    if activation_function == ActivationFunction.SILU:
        return torch.nn.functional.silu
    raise NotImplementedError
