"""Tensor-parallel linear layers.

``ColumnParallelLinear`` shards the output features (weight ``[out / mp, in]``, model-parallel
dimension 0), ``RowParallelLinear`` the input features (weight ``[out, in / mp]``, dimension 1, bias
replicated and added after the reduction).  Constructor arguments, parameter names (``weight``,
``bias`` or ``bias_{bitfit_name}``) and the communication semantics follow the reference
(src/scaling/core/nn/linear/column_parallel_linear.py:29-287, row_parallel_linear.py:37-291).  The
matrix products run on the tcgen05 GEMM of ``scaling_b200.ops`` (forward, dgrad and wgrad) whenever
the tensors live on a GPU.
"""

from __future__ import annotations

from typing import Any, Callable, Optional

import torch

from ....ops import functional as K
from ....parallel.collectives import (
    SequenceShard,
    all_concat,
    all_reduce,
    all_shard,
    copy_to_tensor_model_parallel_region,
)
from ....parallel.topology import Topology
from ..parameter_meta import UMUP_WEIGHT_TYPE, CoreParameterMeta, UMuPParameterMeta
from ..scale import scale_bwd, scale_fwd
from ..umup import UMuParametrization


def get_device(topology: Optional[Topology], device: Optional[torch.device]) -> torch.device:
    """Explicit device wins; else the topology's device; else the current CUDA device or the CPU."""
    if device is not None:
        return device
    if topology is not None:
        return topology.device
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


class _ParallelLinear(torch.nn.Module):
    _shard_dim: int  # which weight dimension is divided over the tensor-parallel group

    def __init__(self, in_features: int, out_features: int, bias: bool, device: Optional[torch.device],
                 dtype: torch.dtype, topology: Optional[Topology],
                 init_method: Callable[[torch.Tensor], torch.Tensor], bitfit_bias_name: Optional[str],
                 umup_weight_type: Optional[UMUP_WEIGHT_TYPE], umup_on_residual: Optional[bool],
                 fp8_config: Optional[Any]) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self._device = get_device(topology, device)
        self.dtype = dtype
        self.topology = topology
        self.init_method = init_method
        self.fp8_config = fp8_config
        self.model_parallel_size = 1 if topology is None else topology.config.model_parallel_size
        mp = self.model_parallel_size
        if self._shard_dim == 0:
            assert out_features % mp == 0, (
                f"cannot column parallelize, out_features ({out_features}) needs to be divisible by "
                f"model parallel size ({mp})"
            )
            w_shape = (out_features // mp, in_features)
            b_shape = (out_features // mp,)
        else:
            assert in_features % mp == 0, (
                f"cannot row parallelize, in_features ({in_features}) needs to be divisible by "
                f"model parallel size ({mp})"
            )
            w_shape = (out_features, in_features // mp)
            b_shape = (out_features,)

        self.load_in_fp8 = bool(
            fp8_config is not None and fp8_config.dtypes_forward is not None and fp8_config.load_in_fp8
        )
        w_dtype = fp8_config.dtypes_forward.right_dtype.torch_dtype if self.load_in_fp8 else dtype
        self.weight = torch.nn.Parameter(torch.empty(w_shape, device=self._device, dtype=w_dtype))
        if not self.load_in_fp8:
            init_method(self.weight)
        CoreParameterMeta.register_on_parameter(self.weight, is_model_parallel=True,
                                                model_parallel_dimension=self._shard_dim)
        self.bias_name: Optional[str] = None
        if bias:
            self.bias_name = "bias" if not bitfit_bias_name else f"bias_{bitfit_bias_name}"
            b = torch.nn.Parameter(torch.zeros(b_shape, device=self._device, dtype=dtype))
            setattr(self, self.bias_name, b)
            if self._shard_dim == 0:
                CoreParameterMeta.register_on_parameter(b, is_model_parallel=True, model_parallel_dimension=0)
            else:
                CoreParameterMeta.register_on_parameter(b, is_model_parallel=False)

        self.umup_weight_type = umup_weight_type
        self.umup_on_residual = umup_on_residual
        self._use_umup = False
        self.forward_multiplier = 1.0
        self.backward_multiplier = 1.0
        self.weight_grad_multiplier = 1.0
        self.bias_grad_multiplier = 1.0

    # ---- helpers
    def _bias(self) -> Optional[torch.Tensor]:
        return getattr(self, self.bias_name) if self.bias_name is not None else None

    def _matmul(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                activation: str = "none") -> torch.Tensor:
        if self.fp8_config is not None:
            assert activation == "none"
            from ...fp8 import fp8_linear

            return fp8_linear(
                x, weight, bias,
                dtypes_forward=self.fp8_config.torch_dtypes_forward,
                dtypes_grad_input=self.fp8_config.torch_dtypes_grad_input,
                dtypes_grad_weight=self.fp8_config.torch_dtypes_grad_weight,
            )
        return K.linear(x, weight, bias, act=activation)

    def _distributed(self) -> bool:
        return self.model_parallel_size > 1 and self.topology is not None and self.topology.is_distributed_initialized

    def umup_setup(self, effective_batch_size: int, depth: int, **kwargs: Any) -> None:
        assert self.umup_weight_type in (UMUP_WEIGHT_TYPE.INPUT_WEIGHT, UMUP_WEIGHT_TYPE.HIDDEN_WEIGHT,
                                         UMUP_WEIGHT_TYPE.OUTPUT_WEIGHT), (
            "when using u-mup, the weight type of the linear layer needs to be provided as input, hidden or output."
        )
        assert isinstance(self.umup_on_residual, bool), (
            "when using u-mup, you need to specify if linear layer is on a residual connection."
        )
        self._use_umup = True
        mp = self.model_parallel_size
        wm: CoreParameterMeta = self.weight.core_parameter_meta  # type: ignore[attr-defined]
        wm.umup_meta = UMuPParameterMeta(weight_type=self.umup_weight_type, on_residual=self.umup_on_residual)
        UMuParametrization.apply_umup_to_weight(self.weight, mp, effective_batch_size, depth,
                                                reinitialize=not self.load_in_fp8)
        self.forward_multiplier = wm.umup_meta.forward_multiplier
        self.backward_multiplier = wm.umup_meta.backward_multiplier
        self.weight_grad_multiplier = wm.umup_meta.grad_multiplier
        b = self._bias()
        if b is not None:
            bm: CoreParameterMeta = b.core_parameter_meta  # type: ignore[attr-defined]
            bm.umup_meta = UMuPParameterMeta(weight_type=UMUP_WEIGHT_TYPE.BIAS, on_residual=self.umup_on_residual)
            UMuParametrization.apply_umup_to_weight(b, mp, effective_batch_size, depth)
            self.bias_grad_multiplier = bm.umup_meta.grad_multiplier

    def _umup_matmul(self, x: torch.Tensor) -> tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Unit-scaled product; returns (scaled output, gradient-scaled bias)."""
        x = scale_bwd(x, self.backward_multiplier)
        w = scale_bwd(self.weight, self.weight_grad_multiplier)
        b = self._bias()
        if b is not None:
            b = scale_bwd(b, self.bias_grad_multiplier)
        return scale_fwd(self._matmul(x, w, None), self.forward_multiplier), b


class ColumnParallelLinear(_ParallelLinear):
    """``Y = X A^T + b`` with ``A`` split along its output features: ``A = [A_1; ...; A_p]``."""

    _shard_dim = 0

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.float32,
                 topology: Optional[Topology] = None,
                 init_method: Callable[[torch.Tensor], torch.Tensor] = torch.nn.init.xavier_normal_,
                 parallel_output: bool = False, bitfit_bias_name: Optional[str] = None,
                 umup_weight_type: Optional[UMUP_WEIGHT_TYPE] = None, umup_on_residual: Optional[bool] = None,
                 fp8_config: Optional[Any] = None):
        super().__init__(in_features, out_features, bias, device, dtype, topology, init_method, bitfit_bias_name,
                         umup_weight_type, umup_on_residual, fp8_config)
        self.parallel_output = parallel_output
        self.output_features_per_partition = self.out_features // self.model_parallel_size

    def forward(self, x: torch.Tensor, activation: str = "none") -> torch.Tensor:
        """``activation="gelu"`` fuses the exact GELU into the GEMM epilogue (parallel output only)."""
        # the backward of the identity below is the all-reduce of dX; in sequence-parallel mode the
        # caller gathers tokens before and reduce-scatters the gradient instead
        if isinstance(x, SequenceShard):
            y = None
            if (self._distributed() and not self._use_umup and self.fp8_config is None
                    and (self.parallel_output or activation == "none")):
                from ....parallel.fused_tp import column_parallel_linear_sp

                y = column_parallel_linear_sp(x.shard, self.weight, self._bias(), activation, self.topology,
                                              list(x.shape))
            if y is not None:
                return y if self.parallel_output else all_concat(y, self.topology)
            x = x.gathered()
        if (self._distributed() and not self.topology.config.sequence_parallel  # type: ignore[union-attr]
                and not self._use_umup and self.fp8_config is None and (self.parallel_output or activation == "none")):
            # the all-reduce of the input gradient runs inside the dgrad GEMM where the group supports it
            from ....parallel.fused_tp import column_parallel_linear

            y = column_parallel_linear(x, self.weight, self._bias(), activation, self.topology)
            if y is not None:
                return y if self.parallel_output else all_concat(y, self.topology)
        if self._distributed() and not self.topology.config.sequence_parallel:  # type: ignore[union-attr]
            x = copy_to_tensor_model_parallel_region(x, self.topology)
        if self._use_umup:
            y, b = self._umup_matmul(x)
            if b is not None:
                y = y + b
        else:
            fuse = activation != "none" and self.fp8_config is None and (self.parallel_output or self.topology is None)
            y = self._matmul(x, self.weight, self._bias(), activation if fuse else "none")
            if activation == "gelu" and not fuse:
                y = K.gelu(y)
            activation = "none"
        if activation == "gelu":
            y = K.gelu(y)
        if self.parallel_output or self.topology is None:
            return y
        return all_concat(y, self.topology)


class RowParallelLinear(_ParallelLinear):
    """``Y = X A^T + b`` with ``A`` split along its input features; partial products are summed."""

    _shard_dim = 1

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.float32,
                 topology: Optional[Topology] = None,
                 init_method: Callable[[torch.Tensor], torch.Tensor] = torch.nn.init.xavier_normal_,
                 parallel_input: bool = False, parallel_output: bool = False,
                 bitfit_bias_name: Optional[str] = None, umup_weight_type: Optional[UMUP_WEIGHT_TYPE] = None,
                 umup_on_residual: Optional[bool] = None, fp8_config: Optional[Any] = None) -> None:
        super().__init__(in_features, out_features, bias, device, dtype, topology, init_method, bitfit_bias_name,
                         umup_weight_type, umup_on_residual, fp8_config)
        self.parallel_input = parallel_input
        self.parallel_output = parallel_output
        self.input_features_per_partition = self.in_features // self.model_parallel_size
        # partial (unreduced) output: the caller reduces it, so the bias may enter only once - it is added on
        # tensor-parallel rank 0, whose bias gradient is then the complete one and is summed over the group
        self._bias_on_first_rank_only = bool(parallel_output and self.model_parallel_size > 1)
        b = self._bias()
        if b is not None and self._bias_on_first_rank_only:
            b.reduce_grad_over_model_parallel = True  # type: ignore[attr-defined]

    def forward_to_sequence_parallel(self, x: torch.Tensor) -> torch.Tensor:
        """``forward`` followed by the reduce-scatter over tokens (sequence parallelism; this layer was built with
        ``parallel_output=True``): one kernel where the group supports it."""
        from ....parallel.collectives import _sp_out_shape, all_reduce_scatter_to_sequence_parallel

        if (self.parallel_input and self.parallel_output and not self._use_umup and self.fp8_config is None
                and self._distributed() and x.dim() == 3):
            from ....parallel.fused_tp import row_parallel_linear_sp

            out_shape = _sp_out_shape(x.shape, self.model_parallel_size, gather=False)
            out_shape[-1] = self.out_features
            y = row_parallel_linear_sp(x, self.weight, self._bias(), self.topology, out_shape)
            if y is not None:
                return y
        return all_reduce_scatter_to_sequence_parallel(self.forward(x), self.topology)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.model_parallel_size > 1 and not self.parallel_input:
            x = all_shard(x, self.topology)
        if self._use_umup:
            y, bias = self._umup_matmul(x)
        elif self.model_parallel_size == 1:
            # nothing is reduced afterwards: the bias goes into the GEMM epilogue
            return self._matmul(x, self.weight, self._bias())
        else:
            if not self.parallel_output and self.fp8_config is None and self._distributed():
                # the all-reduce runs inside the GEMM kernel (peer memory / NVSwitch) where the group supports it
                from ....parallel.fused_tp import row_parallel_linear

                fused = row_parallel_linear(x, self.weight, self._bias(), self.topology)
                if fused is not None:
                    return fused
            y, bias = self._matmul(x, self.weight, None), self._bias()
        if not (self.parallel_output or self.topology is None):
            y = all_reduce(y, self.topology)
        if bias is not None and not (self._bias_on_first_rank_only and self.topology.model_parallel_rank != 0):  # type: ignore[union-attr]
            y = y + bias  # after the reduction (or on one rank only), so that it is added once
        return y
