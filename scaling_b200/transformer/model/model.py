"""Assembly of the transformer: layer specs, the parallel module, parameter groups, the optimizer.

Layer list (src/scaling/transformer/model/model.py:84-181): ``EmbeddingInput``, ``num_layers`` x
``TransformerLayer``, ``LayerNormWrapper``, then ``TransformerLMHead`` or - with weight tying - a
``TransformerLMHeadTied`` sharing ``embedding.weight`` with the input layer, and optionally a
``TransformerEmbeddingHead``.  Weights are drawn from ``N(0, sqrt(2 / (5 h)))``.  Training groups select
parameters by regular expressions on their names; all ranks agree on the resulting groups
(``model.py:217-381``).  Parameters that belong to no group are frozen for real here
(``requires_grad = False``), so their weight-gradient GEMMs and gradient buffers disappear - the
reference keeps computing them.
"""

from __future__ import annotations

import math
import re
from typing import Optional, Sequence, Union

import torch
import torch.distributed as dist

from ...core.logging import logger
from ...core.nn.parallel_module import LayerSpec, ParallelModule, TiedLayerSpec
from ...core.nn.parameter_meta import CoreParameterMeta
from ...core.optimizer import (
    BaseOptimizer,
    Optimizer,
    OptimizerConfig,
    OptimizerParamGroup,
    OptimizerParamGroupConfig,
)
from ...parallel.topology import Topology
from ..context.config import TrainingGroupConfig, TransformerArchitectureConfig
from ..data.text_dataset_batch import TextDatasetBatch
from ..data.utils import remove_cumulative_seq_lengths_padding
from .layers import (
    EmbeddingInput,
    LayerNormWrapper,
    TransformerEmbeddingHead,
    TransformerLayer,
    TransformerLayerIO,
    TransformerLMHead,
    TransformerLMHeadTied,
)

NamedParameterMeta = tuple[str, torch.Tensor, CoreParameterMeta]


def metrics_aggregation_fn(topology: Topology, metrics: list[dict[str, torch.Tensor]]) -> dict[str, torch.Tensor]:
    """Mean over the micro batches of a step, then over data-parallel ranks."""
    out = {}
    for k in metrics[0]:
        v = torch.stack([torch.as_tensor(m[k], dtype=torch.float32, device=topology.device) for m in metrics]).mean()
        if topology.config.data_parallel_size > 1:
            dist.all_reduce(v, group=topology.data_parallel_group)
            v = v / topology.config.data_parallel_size
        out[k] = v
    return out


class TransformerParallelModule(ParallelModule[TransformerLayerIO, TextDatasetBatch]):
    """Strips the variable-length cumulative sequence lengths before a pipe transfer and rebuilds them
    from the fixed-length padded copy afterwards, so that communication shapes never change."""

    def _prepare_for_send(self, tup: tuple) -> tuple:
        names = list(tup[-1])
        if "cumulative_seq_lengths" not in names:
            return tup
        i = names.index("cumulative_seq_lengths")
        values = list(tup[:-1])
        del values[i], names[i]
        return tuple(values + [names])

    def _after_recv(self, tup: tuple) -> tuple:
        names = list(tup[-1])
        if "cumulative_seq_lengths" in names or "cumulative_seq_lengths_padded" not in names:
            return tup
        padded = tup[names.index("cumulative_seq_lengths_padded")]
        values = list(tup[:-1]) + [remove_cumulative_seq_lengths_padding(padded)]
        return tuple(values + [names + ["cumulative_seq_lengths"]])


def get_transformer_layer_specs(architecture_config: TransformerArchitectureConfig, topology: Optional[Topology] = None,
                                device: Optional[torch.device] = None) -> list[LayerSpec]:
    a = architecture_config
    std = math.sqrt(2.0 / (a.hidden_size * 5))

    def init_method(x: torch.Tensor) -> torch.Tensor:
        return torch.nn.init.normal_(x, mean=0.0, std=std)

    if a.umup.enable:
        assert not a.weight_tying, "u-mup and weight tying are not compatible"
    common = dict(architecture_config=a, topology=topology)
    if device is not None and topology is None:
        common["device"] = device
    tied = ["embedding.weight"]
    specs: list[Union[LayerSpec, TiedLayerSpec]] = []
    if a.weight_tying:
        specs.append(TiedLayerSpec(EmbeddingInput, "embedding_tying", tied, init_method=init_method, **common))
    else:
        specs.append(LayerSpec(EmbeddingInput, init_method=init_method, **common))
    for i in range(a.num_layers):
        specs.append(LayerSpec(TransformerLayer, layer_index=i, init_method=init_method, **common))
    specs.append(LayerSpec(LayerNormWrapper, layer_index=a.num_layers, umup_on_residual=False, **common))
    if a.lm_head:
        if a.weight_tying:
            specs.append(TiedLayerSpec(TransformerLMHeadTied, "embedding_tying", tied, init_method=init_method, **common))
        else:
            specs.append(LayerSpec(TransformerLMHead, init_method=init_method, **common))
    if a.embedding_head_config is not None:
        specs.append(LayerSpec(TransformerEmbeddingHead, **common))
    return specs


def init_model(context, use_continuous_recommunication: bool = False) -> TransformerParallelModule:
    a = context.config.transformer_architecture
    model = TransformerParallelModule(
        layer_specs=get_transformer_layer_specs(a, context.topology), topology=context.topology,
        profiler_config=context.config.profiler, use_continuous_recommunication=use_continuous_recommunication,
    )
    if a.umup.enable:
        depth = a.num_layers if a.umup.normalize_depth_to_num_layers else 2 * a.num_layers
        model.umup_setup(
            effective_batch_size=context.config.topology.global_batch_size * a.sequence_length, depth=depth,
            avg_sequence_length=a.sequence_length, allow_non_umup_params=a.umup.allow_non_umup_params,
        )
    return model


# ---------------------------------------------------------------------- training groups
def _first_match(name: str, patterns: Sequence[str]) -> Optional[str]:
    return next((p for p in patterns if re.search(p, name) is not None), None)


def _find_matching_param(key: NamedParameterMeta, data: Sequence[str]) -> Optional[str]:
    """First pattern of ``data`` found in the parameter's name (src/scaling/transformer/model/model.py:360)."""
    return _first_match(key[0], data)


def _filter_by_param(parameters_exclude: Sequence[str], parameter_list: list[NamedParameterMeta]) -> list[NamedParameterMeta]:
    """The parameters whose names match none of the patterns (src/scaling/transformer/model/model.py:354)."""
    return [p for p in parameter_list if _first_match(p[0], parameters_exclude) is None]


def _all_gather_objects(obj):
    if dist.is_initialized() and dist.get_world_size() > 1:
        out = [None] * dist.get_world_size()
        dist.all_gather_object(out, obj)
        return out
    return [obj]


def _extract_parameters(training_groups: list[TrainingGroupConfig], named_parameters_with_meta: list[NamedParameterMeta],
                        allow_missing_params_in_optimizer: bool) -> list[tuple[list[NamedParameterMeta], TrainingGroupConfig]]:
    result = []
    used: dict[str, str] = {}
    for group in training_groups:
        members: list[NamedParameterMeta] = []
        matched: set[str] = set()
        for npm in named_parameters_with_meta:
            if group.parameters_include:
                hit = _first_match(npm[0], group.parameters_include)
                if hit is None:
                    continue
                matched.add(hit)
            if group.parameters_exclude and _first_match(npm[0], group.parameters_exclude) is not None:
                continue
            members.append(npm)
        if group.parameters_include:
            # a pattern may match only on other pipeline stages; it is an error if it matches nowhere
            missing_here = set(group.parameters_include) - matched
            missing_everywhere = set.intersection(*[set(m) for m in _all_gather_objects(missing_here)])
            if missing_everywhere:
                raise ValueError(f"Unmatched finetunable parameters: {missing_everywhere}")
        for name, p, _ in members:
            key = f"{id(p)}"
            if key in used:
                raise ValueError(
                    f"Parameter '{name}' in more then one training_group. Use 'parameters_include' and "
                    f"'parameters_exclude' to ensure no overlap between training groups."
                )
            used[key] = name
        result.append((members, group))
    if not allow_missing_params_in_optimizer:
        unused = {n for n, p, _ in named_parameters_with_meta if f"{id(p)}" not in used}
        if unused:
            raise ValueError(
                f"The following parameters were not added to any optimizer group: {unused}. "
                f"If this is intended, set 'allow_missing_params_in_optimizer'."
            )
    return result


def get_parameter_groups(context, model: TransformerParallelModule) -> list[OptimizerParamGroup]:
    named = model.named_parameters_with_meta()
    extracted = _extract_parameters(context.config.training_groups, named,
                                    context.config.training.allow_missing_params_in_optimizer)
    device = context.topology.device
    counts = torch.tensor([len(members) for members, _ in extracted] + [0], dtype=torch.int64, device=device)
    counts[-1] = counts[:-1].sum()
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(counts, op=dist.ReduceOp.MAX)
    assert int(counts[-1]) > 0 or int(counts[:-1].sum()) > 0, "did not specify any finetuneable parameters on any rank"
    groups = []
    for i, (members, cfg) in enumerate(extracted):
        if int(counts[i]) == 0:
            continue  # empty on every rank
        groups.append(OptimizerParamGroup(
            named_parameters_with_meta=members,
            config=OptimizerParamGroupConfig(
                name=cfg.group_name, weight_decay=cfg.weight_decay,
                independent_weight_decay=cfg.independent_weight_decay,
                learning_rate_scheduler=cfg.learning_rate_scheduler,
            ),
        ))
    sizes = _all_gather_objects(len(groups))
    assert len(set(sizes)) == 1, f"Got different number of optimizer groups on different ranks \n {sizes}"
    assert groups, "Number of optimizer groups is zero"
    trained = {id(p) for members, _ in extracted for _, p, _ in members}
    frozen = 0
    for p in model.parameters():
        if id(p) not in trained and p.requires_grad:
            p.requires_grad_(False)
            frozen += p.numel()
    if frozen:
        logger.info(f"froze {frozen} parameter elements that belong to no training group")
    return groups


def init_optimizer(context, model: TransformerParallelModule,
                   optimizer_config: Optional[OptimizerConfig] = None) -> BaseOptimizer:
    groups = get_parameter_groups(context=context, model=model)
    return Optimizer(
        config=optimizer_config if optimizer_config is not None else context.config.optimizer,
        parameter_groups=groups, topology=context.topology,
        scale_backward_by_grad_acc=not context.config.transformer_architecture.umup.enable,
    )
