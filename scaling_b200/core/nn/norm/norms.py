"""LayerNorm and RMSNorm modules backed by the fused sm_100a kernels.

Parameter names and flags follow the reference (``weight``, ``bias`` or ``bias_{bitfit_name}``;
both replicated over the tensor-parallel group; src/scaling/core/nn/norm/layernorm.py:17-190,
rms_norm.py:19-106).  In sequence-parallel mode the normalised output is all-gathered over tokens
(its backward is the reduce-scatter).  RMSNorm statistics are accumulated in fp32 here, whereas the
reference evaluates ``x * rsqrt(mean(x^2) + eps)`` in the input dtype.
"""

from __future__ import annotations

from enum import Enum
from typing import Any, Optional, Union

import torch
from pydantic import Field

from ....ops import functional as K
from ....parallel.collectives import SequenceShard, gather_from_sequence_parallel_region
from ....parallel.topology import Topology
from ...config import BaseConfig
from ..parameter_meta import UMUP_WEIGHT_TYPE, CoreParameterMeta, UMuPParameterMeta
from ..scale import scale_bwd, scale_fwd
from ..umup import UMuParametrization


class LayerNormOptimizationType(Enum):
    TORCH = "torch"
    FUSED = "fused"


class LayerNormConfig(BaseConfig):
    optimization_type: LayerNormOptimizationType = Field(
        LayerNormOptimizationType.TORCH,
        description="kept for config compatibility; on GPUs the fused sm_100a kernel is always used",
    )
    layernorm_epsilon: float = Field(1.0e-5, description="A value added to the denominator for numerical stability")


class NormType(Enum):
    LAYERNORM = "layernorm"
    RMS = "rms"


class _Norm(torch.nn.Module):
    def __init__(self, topology: Optional[Topology], umup_on_residual: Optional[bool]) -> None:
        super().__init__()
        self.topology = topology
        self.umup_on_residual = umup_on_residual
        self._use_umup = False
        self.forward_multiplier = 1.0
        self.backward_multiplier = 1.0
        self.weight_grad_multiplier = 1.0
        self.bias_grad_multiplier = 1.0
        self.bias_name: Optional[str] = None

    def _setup_param(self, p: torch.Tensor, kind: UMUP_WEIGHT_TYPE, effective_batch_size: int, depth: int) -> UMuPParameterMeta:
        mp = 1 if self.topology is None else self.topology.config.model_parallel_size
        meta: CoreParameterMeta = p.core_parameter_meta  # type: ignore[attr-defined]
        meta.umup_meta = UMuPParameterMeta(weight_type=kind, on_residual=bool(self.umup_on_residual))
        UMuParametrization.apply_umup_to_weight(p, mp, effective_batch_size, depth)
        return meta.umup_meta

    def umup_setup(self, effective_batch_size: int, depth: int, **kwargs: Any) -> None:
        assert isinstance(self.umup_on_residual, bool), (
            "when using u-mup, you need to specify if norm is on a residual connection."
        )
        self._use_umup = True
        um = self._setup_param(self.weight, UMUP_WEIGHT_TYPE.NORM, effective_batch_size, depth)
        self.forward_multiplier = um.forward_multiplier
        self.backward_multiplier = um.backward_multiplier
        self.weight_grad_multiplier = um.grad_multiplier
        if self.bias_name is not None:
            ub = self._setup_param(getattr(self, self.bias_name), UMUP_WEIGHT_TYPE.BIAS, effective_batch_size, depth)
            self.bias_grad_multiplier = ub.grad_multiplier

    def _mark_sequence_parallel(self) -> None:
        """Under sequence parallelism a norm sees only this rank's tokens: its parameter gradients are
        partial and are summed over the tensor-parallel group before the optimizer step."""
        t = self.topology
        if t is not None and t.config.sequence_parallel and t.config.model_parallel_size > 1:
            for p in self.parameters(recurse=False):
                p.reduce_grad_over_model_parallel = True  # type: ignore[attr-defined]

    def _finish(self, y: torch.Tensor) -> torch.Tensor:
        if self._use_umup:
            y = scale_fwd(y, self.forward_multiplier)
        if self.topology is not None and self.topology.config.sequence_parallel:
            if getattr(self, "defer_gather", False) and not self._forward_hooks:
                # the linears behind this norm gather inside their GEMM (or once, on first need)
                return SequenceShard(y, self.topology)  # type: ignore[return-value]
            y = gather_from_sequence_parallel_region(y, self.topology)
        return y


class LayerNorm(_Norm):
    def __init__(self, config: LayerNormConfig, normalized_shape: int, device: Optional[torch.device] = None,
                 dtype: torch.dtype = torch.float32, bitfit_bias_name: Optional[str] = None,
                 topology: Optional[Topology] = None, umup_on_residual: Optional[bool] = None):
        super().__init__(topology, umup_on_residual)
        self.config = config
        self.bias_name = "bias" if not bitfit_bias_name else f"bias_{bitfit_bias_name}"
        self.normalized_shape = torch.Size((normalized_shape,))
        self.weight = torch.nn.Parameter(torch.ones(normalized_shape, device=device, dtype=dtype))
        CoreParameterMeta.register_on_parameter(self.weight, is_model_parallel=False)
        setattr(self, self.bias_name, torch.nn.Parameter(torch.zeros(normalized_shape, device=device, dtype=dtype)))
        CoreParameterMeta.register_on_parameter(getattr(self, self.bias_name), is_model_parallel=False)
        self._mark_sequence_parallel()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, b = self.weight, getattr(self, self.bias_name)
        if self._use_umup:
            x = scale_bwd(x, self.backward_multiplier)
            w = scale_bwd(w, self.weight_grad_multiplier)
            b = scale_bwd(b, self.bias_grad_multiplier)
        return self._finish(K.layer_norm(x, w, b, self.config.layernorm_epsilon))


class RMSNorm(_Norm):
    def __init__(self, dimensions: int, device: Optional[torch.device] = None,
                 config: LayerNormConfig = LayerNormConfig(), dtype: torch.dtype = torch.float32,
                 topology: Optional[Topology] = None, umup_on_residual: Optional[bool] = None) -> None:
        super().__init__(topology, umup_on_residual)
        self.config = config
        self.eps = config.layernorm_epsilon
        self.weight = torch.nn.Parameter(torch.ones(dimensions, dtype=dtype, device=device))
        CoreParameterMeta.register_on_parameter(self.weight, is_model_parallel=False)
        self._mark_sequence_parallel()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.weight
        if self._use_umup:
            x = scale_bwd(x, self.backward_multiplier)
            w = scale_bwd(w, self.weight_grad_multiplier)
        return self._finish(K.rms_norm(x, w, self.eps))


def get_norm(norm_type: NormType, layernorm_config: Optional[LayerNormConfig], dimensions: int,
             device: Optional[torch.device], dtype: torch.dtype, bitfit_bias_name: Optional[str] = None,
             topology: Optional[Topology] = None, umup_on_residual: Optional[bool] = None) -> Union[LayerNorm, RMSNorm]:
    assert layernorm_config is not None
    if norm_type == NormType.LAYERNORM:
        return LayerNorm(config=layernorm_config, normalized_shape=dimensions, device=device, dtype=dtype,
                         bitfit_bias_name=bitfit_bias_name, topology=topology, umup_on_residual=umup_on_residual)
    if norm_type == NormType.RMS:
        return RMSNorm(config=layernorm_config, dimensions=dimensions, device=device, dtype=dtype, topology=topology,
                       umup_on_residual=umup_on_residual)
    raise NotImplementedError(f"{norm_type}")
