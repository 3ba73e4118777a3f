"""FP8 linear settings (fields of src/scaling/core/fp8/fp8_config.py:9-82)."""

from __future__ import annotations

from enum import Enum
from typing import Optional

import torch
from pydantic import Field, model_validator

from ..config import BaseConfig


class FP8DType(str, Enum):
    E4M3 = "e4m3"
    E5M2 = "e5m2"

    @property
    def torch_dtype(self) -> torch.dtype:
        return torch.float8_e4m3fn if self == FP8DType.E4M3 else torch.float8_e5m2


class FP8MatmulConfig(BaseConfig):
    left_dtype: FP8DType = Field(FP8DType.E4M3, description="dtype of the left operand")
    right_dtype: FP8DType = Field(FP8DType.E4M3, description="dtype of the right operand")

    @property
    def torch_dtypes(self) -> tuple[torch.dtype, torch.dtype]:
        return self.left_dtype.torch_dtype, self.right_dtype.torch_dtype

    @model_validator(mode="after")
    def _no_double_e5m2(self) -> "FP8MatmulConfig":
        if self.left_dtype == self.right_dtype == FP8DType.E5M2:
            raise ValueError("Received invalid combination of fp8 dtypes. Cannot multiply two e5m2 tensors.")
        return self


class FP8LinearConfig(BaseConfig):
    dtypes_forward: Optional[FP8MatmulConfig] = Field(
        FP8MatmulConfig(left_dtype=FP8DType.E4M3, right_dtype=FP8DType.E4M3), description="dtypes of (x, w) in forward"
    )
    dtypes_grad_input: Optional[FP8MatmulConfig] = Field(
        FP8MatmulConfig(left_dtype=FP8DType.E5M2, right_dtype=FP8DType.E4M3), description="dtypes of (grad_y, w)"
    )
    dtypes_grad_weight: Optional[FP8MatmulConfig] = Field(
        FP8MatmulConfig(left_dtype=FP8DType.E4M3, right_dtype=FP8DType.E5M2), description="dtypes of (x, grad_y)"
    )
    load_in_fp8: bool = Field(False, description="keep the weights in fp8 (inference); set internally")

    @property
    def torch_dtypes_forward(self) -> Optional[tuple[torch.dtype, torch.dtype]]:
        return None if self.dtypes_forward is None else self.dtypes_forward.torch_dtypes

    @property
    def torch_dtypes_grad_input(self) -> Optional[tuple[torch.dtype, torch.dtype]]:
        return None if self.dtypes_grad_input is None else self.dtypes_grad_input.torch_dtypes

    @property
    def torch_dtypes_grad_weight(self) -> Optional[tuple[torch.dtype, torch.dtype]]:
        return None if self.dtypes_grad_weight is None else self.dtypes_grad_weight.torch_dtypes
