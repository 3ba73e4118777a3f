"""A model as a list of layers, split over pipeline stages (or devices), with per-layer checkpoints.

Each process instantiates only the layers of its own stage (multi-process training, ``topology``
given) or all layers spread over a list of devices (single-process inference, ``devices`` given).
Every parameter and buffer receives a ``CoreParameterMeta`` naming it independently of the layout.

Checkpoint layout (identical to src/scaling/core/nn/parallel_module/partitioned_module.py:246-408):
one file ``model_state_layer_{i}_{LayerClass}.pt`` per global layer index holding tensor-parallel
merged tensors, plus ``..._{group}.pt`` files for parameters whose name contains an entry of
``separate_file_for_parameters``.  Loading searches several directories in order, accepts the legacy
``Luminous*`` class names, can clone ``.bias`` into ``.bias_{name}`` parameters, re-splits for the
current tensor-parallel layout, and applies regex allow-lists for missing / unexpected / ignored keys.
"""

from __future__ import annotations

import re
from pathlib import Path
from typing import Optional, Sequence, Union

import torch

from ....parallel.topology import Topology
from ....parallel.topology_config import PipePartitionMethod
from ...logging import logger
from ...utils.param_merge import merge_parameter, split_parameter
from ..parameter_meta import CoreParameterMeta, UMuPParameterMeta
from .layer_spec import LayerSpec, TiedLayerSpec
from .pipeline_partitioning import (
    PipePartitionCoordinates,
    pipe_partition_balanced,
    pipe_partition_from_indices,
    pipe_partition_uniform,
)
from .tied_layer_index import TiedLayerIndex

legacy_checkpoint_mapping = {
    "TransformerEmbeddingHead": "LuminousEmbeddingHead",
    "EmbeddingInput": "LuminousEmbeddingInput",
    "TransformerLayer": "LuminousLayer",
    "TransformerLayerIO": "LuminousLayerIO",
    "TransformerLMHead": "LuminousLMHead",
    "TransformerLMHeadTied": "LuminousLMHeadTied",
}


def key_match(key: str, list_of_patterns: list[str]) -> bool:
    return any(re.search(p, key) is not None for p in list_of_patterns)


def _partition_keys(keys: set[str], patterns: list[str]) -> tuple[set[str], set[str]]:
    """(keys matching none of the patterns, keys matching one)."""
    hit = {k for k in keys if key_match(k, patterns)}
    return keys - hit, hit


def _is_legacy_checkpoint(paths: Sequence[Path]) -> bool:
    return any(any(p.glob(f"*{legacy}.pt")) for p in paths for legacy in legacy_checkpoint_mapping.values())


def _named_tensors(layer: torch.nn.Module):
    yield from layer.named_parameters()
    yield from layer.named_buffers()


class PipePartitionedModule(torch.nn.Module):
    def __init__(self, layer_specs: list[LayerSpec], devices: Optional[Sequence[Union[int, str, torch.device]]] = None,
                 topology: Optional[Topology] = None, pipe_partition_method: Optional[PipePartitionMethod] = None,
                 pipe_partition_overwrite: Optional[list[int]] = None):
        super().__init__()
        assert (devices is None) ^ (topology is None), "Exactly either one of 'devices' or 'topology' must be specified"
        self.topology = topology
        self.devices: Optional[list[torch.device]] = None
        if devices is not None:
            self.devices = [d if isinstance(d, torch.device) else
                            (torch.device("cuda", d) if isinstance(d, int) else torch.device(d)) for d in devices]
        self._layer_specs = layer_specs
        if topology is None:
            self.pipe_partition_method = pipe_partition_method or PipePartitionMethod.UNIFORM
            self.pipe_partition_overwrite = pipe_partition_overwrite
        else:
            assert pipe_partition_method is None, "pipe partition method should be provided through the topology"
            assert pipe_partition_overwrite is None, "pipe partition overwrite should be provided through the topology"
            self.pipe_partition_method = topology.config.pipe_partition_method
            self.pipe_partition_overwrite = topology.config.pipe_partition_overwrite
        self._initialize_layers()

    # ------------------------------------------------------------------ construction
    def _get_pipe_partition_coordinates(self) -> list[PipePartitionCoordinates]:
        parts = len(self.devices) if self.devices is not None else self.topology.config.pipe_parallel_size  # type: ignore[union-attr]
        n = len(self._layer_specs)
        if n < parts:
            raise RuntimeError(f"Number of layers ({n}) is smaller than number of pipe partitions {parts}")
        if self.pipe_partition_overwrite is not None:
            return pipe_partition_from_indices(self.pipe_partition_overwrite, num_layers=n)
        if self.pipe_partition_method == PipePartitionMethod.UNIFORM:
            return pipe_partition_uniform(item_count=n, partition_count=parts)
        if self.pipe_partition_method == PipePartitionMethod.BALANCED:
            return pipe_partition_balanced(layer_specs=self._layer_specs, partition_count=parts)
        raise NotImplementedError(f"Pipe partition method not known: {self.pipe_partition_method}")

    def _initialize_layers(self) -> None:
        coords = self._get_pipe_partition_coordinates()
        for stage, c in enumerate(coords):
            assert c.start < c.end, f"no parallel module layer spec assigned to index {stage}"
            if self.topology is None or self.topology.config.global_rank == 0:
                logger.debug(f"pipe_parallel_rank {stage} gets layers {c.start}:{c.end}")
        self._all_pipe_partition_coordinates = coords
        if self.topology is not None:
            self._pipe_partition_coordinates = [coords[self.topology.pipe_parallel_rank]]
            devices = [self.topology.device]
            self.tied_layer_index: Optional[TiedLayerIndex] = TiedLayerIndex(
                pipe_partition_coordinates=coords, layer_specs=self._layer_specs, topology=self.topology,
                device=self.topology.device,
            )
        else:
            self._pipe_partition_coordinates = coords
            devices = self.devices  # type: ignore[assignment]
            self.tied_layer_index = None
        self._layers = torch.nn.ModuleList()
        self._layer_devices: list[torch.device] = []
        for device, c in zip(devices, self._pipe_partition_coordinates):
            for layer_index in range(c.start, c.end):
                spec = self._layer_specs[layer_index]
                tied_attrs: set[str] = set()
                if isinstance(spec, TiedLayerSpec):
                    assert self.tied_layer_index is not None, (
                        "TiedLayerSpecs are currently only supported when providing a topology"
                    )
                    layer = self.tied_layer_index.get_module_by_layer_index(layer_index)
                    tied_attrs = self.tied_layer_index.get_tied_weight_attributes_by_layer_index(layer_index)
                else:
                    layer = spec.initialize(device=device)
                cls_name = type(layer).__name__
                for name, tensor in _named_tensors(layer):
                    tied = name in tied_attrs
                    if hasattr(tensor, "core_parameter_meta"):
                        tensor.core_parameter_meta.set(layer_index=layer_index, parameter_name=name,
                                                       layer_class_name=cls_name, is_tied=tied)
                    else:
                        CoreParameterMeta.register_on_parameter(
                            tensor, is_model_parallel=False, layer_index=layer_index, parameter_name=name,
                            layer_class_name=cls_name, is_tied=tied,
                        )
                self._layers.append(layer)
                self._layer_devices.append(device)

    @property
    def first_layer_index(self) -> int:
        return self._pipe_partition_coordinates[0].start

    # ------------------------------------------------------------------ u-muP
    def umup_setup(self, effective_batch_size: int, depth: int, avg_sequence_length: int,
                   allow_non_umup_params: bool = False) -> None:
        for module in self.modules():
            if module is self or not hasattr(module, "umup_setup"):
                continue
            module.umup_setup(effective_batch_size=effective_batch_size, depth=depth,
                              avg_sequence_length=avg_sequence_length)
            assert getattr(module, "_use_umup", False), type(module)
        if allow_non_umup_params:
            return
        for n, p in self.named_parameters():
            meta = getattr(p, "core_parameter_meta", None)
            assert isinstance(meta, CoreParameterMeta)
            assert isinstance(meta.umup_meta, UMuPParameterMeta), f"mup parameter meta not set for {n}"

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, dir_: Union[Path, str], separate_file_for_parameters: Optional[list[str]] = None) -> None:
        if self.topology is not None and self.topology.data_parallel_rank != 0:
            return
        dir_ = Path(dir_)
        dir_.mkdir(parents=True, exist_ok=True)
        groups = list(separate_file_for_parameters or [])
        writer = self.topology is None or self.topology.model_parallel_rank == 0
        for local_index, layer in enumerate(self._layers):
            layer_index = self._global_layer_index(local_index)
            persistent = set(layer.state_dict().keys())
            files: dict[str, dict[str, torch.Tensor]] = {"": {}}
            for name, tensor in _named_tensors(layer):
                if name not in persistent:  # non-persistent buffers
                    continue
                meta: CoreParameterMeta = tensor.core_parameter_meta  # type: ignore[attr-defined]
                merged = merge_parameter(tensor, meta, self.topology) if self.topology is not None else tensor.detach().clone().cpu()
                group = ""
                for g in groups:
                    if g in name:
                        group = g
                files.setdefault(group, {})[name] = merged
            if not writer:
                continue
            for group, state in files.items():
                if not state:
                    continue
                suffix = f"_{group}" if group else ""
                torch.save(state, str(dir_ / f"model_state_layer_{layer_index}_{type(layer).__name__}{suffix}.pt"))

    def _global_layer_index(self, local_index: int) -> int:
        if self.topology is not None:
            return self._pipe_partition_coordinates[0].start + local_index
        return local_index  # single process: all layers are local, in order

    def load_checkpoint(self, dir_: Union[Path, str, list], add_bias_names_if_not_exist: Optional[list[str]] = None,
                        add_bias_names_if_not_exist_exceptions: Optional[list[str]] = None,
                        allowed_missing_keys_in_checkpoint: Optional[list[str]] = None,
                        allowed_unexpected_keys_in_checkpoint: Optional[list[str]] = None,
                        ignore_keys_in_checkpoint: Optional[list[str]] = None) -> None:
        paths = [Path(p) for p in (dir_ if isinstance(dir_, list) else [dir_])]
        missing_dirs = [p for p in paths if not p.is_dir()]
        if missing_dirs:
            raise RuntimeError(f"Weight set directories missing: {missing_dirs}")
        legacy = _is_legacy_checkpoint(paths)
        allowed_missing = list(allowed_missing_keys_in_checkpoint or [])
        ignore = list(ignore_keys_in_checkpoint or [])
        allowed_unexpected = list(allowed_unexpected_keys_in_checkpoint or []) + ignore
        unexpected: set[str] = set()
        missing: set[str] = set()
        for local_index, layer in enumerate(self._layers):
            layer_index = self._global_layer_index(local_index)
            cls_name = type(layer).__name__
            if legacy:
                cls_name = legacy_checkpoint_mapping.get(cls_name, cls_name)
            state: dict[str, torch.Tensor] = {}
            for p in paths:
                for f in sorted(p.glob(f"model_state_layer_{layer_index}_{cls_name}*.pt")):
                    state.update(torch.load(f, map_location="cpu", weights_only=False))
            for k in list(state.keys()) if add_bias_names_if_not_exist else []:
                if not k.endswith(".bias"):
                    continue
                if add_bias_names_if_not_exist_exceptions and any(
                        part == e for part in k.split(".") for e in add_bias_names_if_not_exist_exceptions):
                    continue
                for bias_name in add_bias_names_if_not_exist or []:
                    if bias_name and f"{k}_{bias_name}" not in state:
                        state[f"{k}_{bias_name}"] = state[k].clone()
            if self.topology is not None and self.topology.config.model_parallel_size > 1:
                for name, tensor in _named_tensors(layer):
                    meta: CoreParameterMeta = tensor.core_parameter_meta  # type: ignore[attr-defined]
                    if name in state and meta.is_model_parallel:
                        state[name] = split_parameter(state[name].data, meta, self.topology)
            if ignore:
                state = {k: v for k, v in state.items() if not key_match(k, ignore)}
            result = layer.load_state_dict(state, strict=False)
            missing.update(result.missing_keys)
            unexpected.update(result.unexpected_keys)
        bad_unexpected, ok_unexpected = _partition_keys(unexpected, allowed_unexpected)
        if ok_unexpected:
            logger.warning(f"Ignoring unexpected keys in checkpoint: {ok_unexpected}")
        if bad_unexpected:
            raise RuntimeError(f"Unexpected keys in checkpoint: {bad_unexpected}. You may add keys to "
                               f"'allowed_unexpected_keys_in_checkpoint'.")
        bad_missing, ok_missing = _partition_keys(missing, allowed_missing)
        if ok_missing:
            logger.warning(f"Ignoring missing keys in checkpoint: {ok_missing}")
        if bad_missing:
            raise RuntimeError(f"Missing keys in checkpoint: {bad_missing}. You may add keys to "
                               f"'allowed_missing_keys_in_checkpoint'.")
