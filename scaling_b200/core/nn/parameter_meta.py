"""Identity record attached to every parameter (``param.core_parameter_meta``).

It names the parameter independently of the parallel layout - layer index, attribute path, whether
and along which dimension it is sharded over the tensor-parallel group - which is what makes model
and optimizer checkpoints layout independent.  Attribute names and the ``key`` format follow the
reference (src/scaling/core/nn/parameter_meta.py:44-193) so that its checkpoints load unchanged.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Optional

import torch


class UMUP_WEIGHT_TYPE(str, Enum):
    INPUT_WEIGHT = "input_weight"
    HIDDEN_WEIGHT = "hidden_weight"
    OUTPUT_WEIGHT = "output_weight"
    INPUT_EMBEDDING = "embedding"
    BIAS = "bias"
    NORM = "norm"


@dataclass
class UMuPParameterMeta:
    weight_type: UMUP_WEIGHT_TYPE
    on_residual: bool
    forward_multiplier: float = 1.0
    backward_multiplier: float = 1.0
    grad_multiplier: float = 1.0
    lr_multiplier: float = 1.0


@dataclass(eq=False)
class CoreParameterMeta:
    local_shape: tuple[int, ...]
    is_model_parallel: bool
    model_parallel_dimension: Optional[int] = None
    layer_index: Optional[int] = None
    parameter_name: Optional[str] = None
    layer_class_name: Optional[str] = None
    is_tied: bool = False
    tied_layer_indices: set[int] = field(default_factory=set)
    tied_grad_on_model_parallel: bool = False
    lr_gain: float = 1.0
    umup_meta: Optional[UMuPParameterMeta] = None

    def __post_init__(self) -> None:
        if self.tied_layer_indices is None:
            self.tied_layer_indices = set()
        else:
            self.tied_layer_indices = set(self.tied_layer_indices)
        if self.layer_index is not None:
            self.set_layer_index(self.layer_index)

    # ---- identity
    def key_for_layer(self, layer_index: int) -> str:
        return (
            f"layer_index_{layer_index}_parameter_name_{self.parameter_name}_"
            f"is_model_parallel_{self.is_model_parallel}_"
            f"model_parallel_dimension_{self.model_parallel_dimension}"
        )

    @property
    def key(self) -> str:
        """Unique within one architecture, independent of the parallel layout."""
        return self.key_for_layer(self.layer_index)  # type: ignore[arg-type]

    def possible_keys(self) -> list[str]:
        if self.is_tied:
            return [self.key_for_layer(i) for i in sorted(self.tied_layer_indices)]
        return [self.key]

    @property
    def is_model_parallel_duplicate(self) -> bool:
        """True for parameters replicated on every tensor-parallel rank."""
        return not self.is_model_parallel

    def __eq__(self, other: Any) -> bool:
        return isinstance(other, CoreParameterMeta) and self.key == other.key

    def __hash__(self) -> int:
        return hash(self.key)

    def __repr__(self) -> str:
        return (
            f"CoreParameterMeta [{self.parameter_name}] layer_index [{self.layer_index}] "
            f"layer_class_name [{self.layer_class_name}] is_model_parallel [{self.is_model_parallel}]"
        )

    # ---- mutation helpers
    def scale_lr_gain(self, factor: float) -> None:
        self.lr_gain *= factor

    def set_layer_index(self, layer_index: int) -> None:
        self.layer_index = layer_index
        if self.is_tied:
            self.tied_layer_indices.add(layer_index)

    def set_parameter_name(self, parameter_name: str) -> None:
        self.parameter_name = parameter_name

    def set_layer_class_name(self, layer_class_name: str) -> None:
        self.layer_class_name = layer_class_name

    def set_is_tied(self, is_tied: bool) -> None:
        self.is_tied = is_tied

    def set(self, layer_index: int, parameter_name: str, layer_class_name: str, is_tied: bool) -> None:
        self.set_is_tied(is_tied)
        self.set_layer_index(layer_index)
        self.set_parameter_name(parameter_name)
        self.set_layer_class_name(layer_class_name)

    # ---- (de)serialisation
    def state_dict(self) -> dict[str, Any]:
        return {
            "local_shape": tuple(self.local_shape),
            "is_model_parallel": self.is_model_parallel,
            "model_parallel_dimension": self.model_parallel_dimension,
            "layer_index": self.layer_index,
            "parameter_name": self.parameter_name,
            "is_tied": self.is_tied,
            "tied_layer_indices": set(self.tied_layer_indices),
            "tied_grad_on_model_parallel": self.tied_grad_on_model_parallel,
            "lr_gain": self.lr_gain,
            "umup_meta": self.umup_meta,
        }

    @classmethod
    def from_state_dict(cls, state_dict: dict[str, Any]) -> "CoreParameterMeta":
        d = dict(state_dict)
        d["local_shape"] = tuple(d["local_shape"])
        d["tied_layer_indices"] = set(d.get("tied_layer_indices") or ())
        d.pop("layer_class_name", None)
        return cls(**d)

    @staticmethod
    def register_on_parameter(
        parameter: torch.Tensor,
        is_model_parallel: bool,
        model_parallel_dimension: Optional[int] = None,
        layer_index: Optional[int] = None,
        parameter_name: Optional[str] = None,
        layer_class_name: Optional[str] = None,
        is_tied: bool = False,
        tied_grad_on_model_parallel: bool = False,
    ) -> "CoreParameterMeta":
        assert not hasattr(parameter, "core_parameter_meta"), "core_parameter_meta already registered"
        meta = CoreParameterMeta(
            local_shape=tuple(parameter.shape),
            is_model_parallel=is_model_parallel,
            model_parallel_dimension=model_parallel_dimension,
            layer_index=layer_index,
            parameter_name=parameter_name,
            layer_class_name=layer_class_name,
            is_tied=is_tied,
            tied_grad_on_model_parallel=tied_grad_on_model_parallel,
        )
        parameter.core_parameter_meta = meta  # type: ignore[attr-defined]
        return meta
