"""MLP classifier built from tensor-parallel linears on the core engine:
``Column(in -> h) ReLU [Row(h -> h) ReLU Column(h -> h) ReLU ...] -> classes`` with column- and
row-parallel layers alternating, as in the reference example (examples/mlp_example/model.py:126-155)."""

from __future__ import annotations

from typing import Any, Callable

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ...core.context import BaseContext
from ...core.data import BaseLayerIO
from ...core.nn.linear import ColumnParallelLinear, RowParallelLinear
from ...core.nn.parallel_module import BaseLayer, LayerSpec, ParallelModule
from ...core.optimizer import BaseOptimizer, Optimizer, OptimizerParamGroup, OptimizerParamGroupConfig
from ...parallel.topology import Topology
from .config import MLPConfig
from .data import MLPDatasetBatch

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


class MLPContext(BaseContext):
    config: MLPConfig


class MLPLayerIO(BaseLayerIO):
    def __init__(self, activations: torch.Tensor):
        self.activations = activations


def _identity(x: torch.Tensor) -> torch.Tensor:
    return x


class MLPBaseLayer(BaseLayer[MLPLayerIO, MLPLayerIO, MLPLayerIO]):
    linear: torch.nn.Module
    act_fn: Callable

    @staticmethod
    def input_to_tuple(input: Any) -> tuple[Any, ...]:
        return (input.activations if isinstance(input, MLPLayerIO) else input.inputs,)

    @staticmethod
    def tuple_to_input(d: tuple[Any, ...]) -> MLPLayerIO:
        return MLPLayerIO(activations=d[0])

    @staticmethod
    def output_to_tuple(output: MLPLayerIO) -> tuple[Any, ...]:
        return (output.activations,)

    @staticmethod
    def tuple_to_last_stage_activation(d: tuple[Any, ...]) -> MLPLayerIO:
        return MLPLayerIO(activations=d[0])

    def forward(self, x: Any) -> MLPLayerIO:
        inp = x.activations if isinstance(x, MLPLayerIO) else x.inputs
        h = torch.flatten(inp, start_dim=1).to(self.linear.weight.dtype)
        return MLPLayerIO(activations=self.act_fn(self.linear(h)))


class MLPLinearColumnParallel(MLPBaseLayer):
    def __init__(self, in_features: int, out_features: int, topology: Topology, parallel_output: bool = True,
                 act_fn: Callable = _identity, dtype: torch.dtype = torch.float32):
        super().__init__()
        self.linear = ColumnParallelLinear(in_features=in_features, out_features=out_features,
                                           parallel_output=parallel_output, topology=topology, dtype=dtype, bias=True)
        self.act_fn = act_fn


class MLPLinearRowParallel(MLPBaseLayer):
    def __init__(self, in_features: int, out_features: int, topology: Topology, act_fn: Callable = _identity,
                 dtype: torch.dtype = torch.float32, parallel_input: bool = True):
        super().__init__()
        self.linear = RowParallelLinear(in_features=in_features, out_features=out_features,
                                        parallel_input=parallel_input, topology=topology, dtype=dtype, bias=True)
        self.act_fn = act_fn


def loss_function(output: MLPLayerIO, batch: MLPDatasetBatch) -> tuple[torch.Tensor, dict[str, torch.Tensor]]:
    logits = output.activations.float()
    targets = batch.targets.to(torch.long)
    loss = F.cross_entropy(logits, targets)
    accuracy = (logits.argmax(dim=1) == targets).float().mean()
    return loss, {"accuracy": accuracy}


def metrics_aggregation_fn(topology: Topology, metrics: list[dict[str, torch.Tensor]]) -> dict[str, torch.Tensor]:
    out = {}
    for k in metrics[0]:
        v = torch.stack([torch.as_tensor(m[k], dtype=torch.float32, device=topology.device) for m in metrics]).mean()
        if topology.config.data_parallel_size > 1:
            dist.all_reduce(v, group=topology.data_parallel_group)
            v = v / topology.config.data_parallel_size
        out[k] = v
    return out


def get_layer_specs(config: MLPConfig, topology: Topology) -> list[LayerSpec]:
    a = config.architecture
    dtype = _DTYPES[a.precision]
    n_layers = a.n_hidden_layers + 2
    specs = []
    for i in range(n_layers):
        last = i == n_layers - 1
        kwargs: dict[str, Any] = dict(
            in_features=a.input_dim if i == 0 else a.hidden_dim,
            out_features=a.output_dim if last else a.hidden_dim,
            topology=topology, dtype=dtype,
        )
        if not last:
            kwargs["act_fn"] = F.relu
        if i % 2 == 0:
            if last:
                kwargs["parallel_output"] = False
            specs.append(LayerSpec(MLPLinearColumnParallel, **kwargs))
        else:
            specs.append(LayerSpec(MLPLinearRowParallel, **kwargs))
    return specs


def init_model(context: MLPContext) -> ParallelModule:
    return ParallelModule(layer_specs=get_layer_specs(context.config, context.topology), topology=context.topology,
                          profiler_config=context.config.profiler)


def init_optimizer(context: MLPContext, model: ParallelModule) -> BaseOptimizer:
    group = OptimizerParamGroup(
        named_parameters_with_meta=list(model.named_parameters_with_meta()),
        config=OptimizerParamGroupConfig(
            name="weight_decay_params", weight_decay=context.config.training.weight_decay,
            learning_rate_scheduler=context.config.learning_rate_scheduler,
        ),
    )
    return Optimizer(config=context.config.optimizer, parameter_groups=[group], topology=context.topology)
