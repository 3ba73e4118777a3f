"""Tensor-parallel feed-forward blocks.

``ParallelMLP``: column-parallel ``dense_in`` -> GELU (exact) or SiLU -> row-parallel ``dense_out``.
``ParallelSwiGLUMLP``: ``dense_out(silu(dense_in(x)) * siglu_weight(x))`` with two separate
column-parallel input projections, as in the reference (src/scaling/core/nn/mlp.py:25-282), whose
parameter names are kept for checkpoint compatibility.  In sequence-parallel mode the row-parallel
output stays partial and is reduce-scattered over tokens.  On GPUs the GELU runs in the epilogue of
the tcgen05 GEMM and ``silu(a) * g`` is one fused kernel.
"""

from __future__ import annotations

from typing import Any, Callable, Optional

import torch

from ...ops import functional as K
from ...parallel.topology import Topology
from .activation_function import ActivationFunction, get_activation_function
from .linear import ColumnParallelLinear, RowParallelLinear
from .parameter_meta import UMUP_WEIGHT_TYPE
from .scale import scale_bwd, scale_fwd
from .umup import UMuParametrization


def _intermediate(io_features: int, factor: float) -> int:
    n = io_features * factor
    assert float(int(n)) == n, (
        "io_features * intermediate_feature_factor does not result in a natural number for feature dimensions"
    )
    return int(n)


def _umup_types(first: Optional[bool], last: Optional[bool]):
    t_in = t_out = None
    if isinstance(first, bool):
        t_in = UMUP_WEIGHT_TYPE.INPUT_WEIGHT if first else UMUP_WEIGHT_TYPE.HIDDEN_WEIGHT
    if isinstance(last, bool):
        t_out = UMUP_WEIGHT_TYPE.OUTPUT_WEIGHT if last else UMUP_WEIGHT_TYPE.HIDDEN_WEIGHT
    return t_in, t_out


class _MLPBase(torch.nn.Module):
    def __init__(self, topology: Optional[Topology], umup_mult: Optional[float]) -> None:
        super().__init__()
        self.topology = topology
        self.umup_mult = umup_mult
        self._use_umup = False
        self.output_scale_factor = 1.0

    def _project_out(self, x: torch.Tensor) -> torch.Tensor:
        if self.topology is not None and self.topology.config.sequence_parallel:
            return self.dense_out.forward_to_sequence_parallel(x)
        return self.dense_out(x)


class ParallelMLP(_MLPBase):
    def __init__(self, io_features: int, intermediate_feature_factor: float, bias: bool = True,
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.float32,
                 topology: Optional[Topology] = None,
                 init_method: Callable[[torch.Tensor], torch.Tensor] = torch.nn.init.xavier_normal_,
                 bitfit_bias_name: Optional[str] = None,
                 activation_function: ActivationFunction = ActivationFunction.GELU, umup_mult: Optional[float] = None,
                 umup_is_first_layer: Optional[bool] = None, umup_is_last_layer: Optional[bool] = None,
                 umup_on_residual: Optional[bool] = None, fp8_config: Optional[Any] = None,
                 fp8_config_dense_out: Optional[Any] = None) -> None:
        super().__init__(topology, umup_mult)
        inter = _intermediate(io_features, intermediate_feature_factor)
        t_in, t_out = _umup_types(umup_is_first_layer, umup_is_last_layer)
        sp = topology.config.sequence_parallel if topology is not None else False
        self.dense_in = ColumnParallelLinear(
            in_features=io_features, out_features=inter, bias=bias, device=device, dtype=dtype, topology=topology,
            init_method=init_method, parallel_output=True, bitfit_bias_name=bitfit_bias_name, umup_weight_type=t_in,
            umup_on_residual=umup_on_residual, fp8_config=fp8_config,
        )
        self.dense_out = RowParallelLinear(
            in_features=inter, out_features=io_features, bias=bias, device=device, dtype=dtype, topology=topology,
            init_method=init_method, parallel_input=True, parallel_output=sp, bitfit_bias_name=bitfit_bias_name,
            umup_weight_type=t_out, umup_on_residual=umup_on_residual, fp8_config=fp8_config_dense_out,
        )
        self.activation_function_type = activation_function
        self.activation_function = get_activation_function(activation_function)

    def umup_setup(self, **kwargs: Any) -> None:
        assert self.umup_mult is not None
        if self.activation_function_type != ActivationFunction.GELU:
            raise NotImplementedError(
                f"UMuP currently not implemented for activation function {self.activation_function_type}."
            )
        self._use_umup = True
        self.output_scale_factor = UMuParametrization.get_umup_gelu_scales(self.umup_mult)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._use_umup:
            h = scale_bwd(self.dense_in(x), self.output_scale_factor)
            # gelu(x) = x * Phi(x); only Phi takes the temperature
            h = K.gelu(h) if self.umup_mult == 1.0 else K.gelu(self.umup_mult * h) / self.umup_mult
            h = scale_fwd(h, self.output_scale_factor)
        elif self.activation_function_type == ActivationFunction.GELU:
            h = self.dense_in(x, activation="gelu")
        else:
            h = self.activation_function(self.dense_in(x))
        return self._project_out(h)


class ParallelSwiGLUMLP(_MLPBase):
    def __init__(self, io_features: int, intermediate_feature_factor: float, bias: bool = True,
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.float32,
                 topology: Optional[Topology] = None,
                 init_method: Callable[[torch.Tensor], torch.Tensor] = torch.nn.init.xavier_normal_,
                 bitfit_bias_name: Optional[str] = None, umup_mult: Optional[float] = None,
                 umup_is_first_layer: Optional[bool] = None, umup_is_last_layer: Optional[bool] = None,
                 umup_on_residual: Optional[bool] = None, fp8_config: Optional[Any] = None,
                 fp8_config_dense_out: Optional[Any] = None) -> None:
        super().__init__(topology, umup_mult)
        inter = _intermediate(io_features, intermediate_feature_factor)
        t_in, t_out = _umup_types(umup_is_first_layer, umup_is_last_layer)
        sp = topology.config.sequence_parallel if topology is not None else False
        col = dict(in_features=io_features, out_features=inter, bias=bias, device=device, dtype=dtype,
                   topology=topology, init_method=init_method, parallel_output=True,
                   bitfit_bias_name=bitfit_bias_name, umup_weight_type=t_in, umup_on_residual=umup_on_residual,
                   fp8_config=fp8_config)
        self.dense_in = ColumnParallelLinear(**col)
        self.siglu_weight = ColumnParallelLinear(**col)
        self.dense_out = RowParallelLinear(
            in_features=inter, out_features=io_features, bias=bias, device=device, dtype=dtype, topology=topology,
            init_method=init_method, parallel_input=True, parallel_output=sp, bitfit_bias_name=bitfit_bias_name,
            umup_weight_type=t_out, umup_on_residual=umup_on_residual, fp8_config=fp8_config_dense_out,
        )

    def umup_setup(self, **kwargs: Any) -> None:
        assert self.umup_mult is not None
        self._use_umup = True
        self.output_scale_factor = UMuParametrization.get_umup_swiglu_scales(self.umup_mult)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        a, g = self.dense_in(x), self.siglu_weight(x)
        if self._use_umup:
            a = scale_bwd(a, self.output_scale_factor)
            g = scale_bwd(g, self.output_scale_factor)
            m = float(self.umup_mult)
            # silu(x) = x * sigmoid(x); only the sigmoid takes the temperature
            h = K.swiglu(a, g) if m == 1.0 else K.swiglu(a * m, g, scale=1.0 / m)
            h = scale_fwd(h, self.output_scale_factor)
        else:
            h = K.swiglu(a, g)
        return self._project_out(h)
