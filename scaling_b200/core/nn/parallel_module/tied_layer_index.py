"""Bookkeeping for layers that share parameters (e.g. embedding <-> LM head).

For every tie ``key`` it records which layers and pipeline stages hold a copy, builds one process
group per (data, model) coordinate spanning those stages, and makes local duplicates share the
very same ``Parameter`` object.  The engine uses it to broadcast tied weights at start-up, to
all-reduce their gradients every step, and to avoid double counting / double optimisation
(semantics of src/scaling/core/nn/parallel_module/tied_layer_index.py:11-224).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch
import torch.distributed as dist

from ....parallel.topology import Topology
from .layer_spec import LayerSpec, TiedLayerSpec
from .pipeline_partitioning import PipePartitionCoordinates


@dataclass
class TieRecord:
    layer_indices: list[int] = field(default_factory=list)
    pipe_parallel_ranks: set[int] = field(default_factory=set)
    tied_weight_attributes: set[str] = field(default_factory=set)
    is_local: bool = False
    process_group: Any = None
    global_ranks: Optional[list[int]] = None


@dataclass
class TiedModule:
    module: torch.nn.Module
    is_main: bool          # first layer of the tie in the whole model
    is_local_main: bool    # first layer of the tie on this pipeline stage
    tied_weight_attributes: set[str]


def _resolve(module: torch.nn.Module, dotted: str) -> tuple[torch.nn.Module, str]:
    *path, leaf = dotted.split(".")
    for name in path:
        module = getattr(module, name)
    return module, leaf


class TiedLayerIndex:
    def __init__(self, pipe_partition_coordinates: list[PipePartitionCoordinates], layer_specs: list[LayerSpec],
                 topology: Topology, device: Optional[torch.device] = None) -> None:
        own = pipe_partition_coordinates[topology.pipe_parallel_rank]
        stage_of = {}
        for stage, coord in enumerate(pipe_partition_coordinates):
            for i in range(coord.start, coord.end):
                stage_of[i] = stage
        self.layer_index_to_pipe_parallel_rank = stage_of

        # 1. which layers / stages take part in which tie
        self.records: dict[str, TieRecord] = {}
        for i, spec in enumerate(layer_specs):
            if not isinstance(spec, TiedLayerSpec):
                continue
            rec = self.records.setdefault(spec.key, TieRecord())
            rec.layer_indices.append(i)
            rec.pipe_parallel_ranks.add(stage_of[i])
            rec.tied_weight_attributes.update(spec.tied_weight_attributes)
            rec.is_local = rec.is_local or (own.start <= i < own.end)

        # 2. process groups: every rank creates every group, in sorted key order
        for key in sorted(self.records):
            rec = self.records[key]
            for d in range(topology.config.data_parallel_size):
                for m in range(topology.config.model_parallel_size):
                    ranks = sorted(
                        topology.get_global_rank(pipe_parallel_rank=p, data_parallel_rank=d, model_parallel_rank=m)
                        for p in rec.pipe_parallel_ranks
                    )
                    group = dist.new_group(ranks) if len(ranks) > 1 and topology.is_distributed_initialized else None
                    if topology.config.global_rank in ranks:
                        rec.process_group = group
                        rec.global_ranks = ranks

        # 3. instantiate local tied layers; later copies adopt the first copy's Parameter objects
        self.tied_modules_by_layer_index: dict[int, TiedModule] = {}
        self.tied_parameters_by_key: dict[str, dict[str, torch.nn.Parameter]] = {}
        self._local_main: dict[str, TiedModule] = {}
        seen: set[str] = set()
        for i, spec in enumerate(layer_specs):
            if not isinstance(spec, TiedLayerSpec):
                continue
            is_main = spec.key not in seen
            seen.add(spec.key)
            if not (own.start <= i < own.end):
                continue
            is_local_main = spec.key not in self._local_main
            tm = TiedModule(spec.initialize(device), is_main, is_local_main, set(spec.tied_weight_attributes))
            if is_local_main:
                self._local_main[spec.key] = tm
                wanted = self.records[spec.key].tied_weight_attributes
                self.tied_parameters_by_key[spec.key] = {n: p for n, p in tm.module.named_parameters() if n in wanted}
            else:
                main = self._local_main[spec.key].module
                for attr in spec.tied_weight_attributes:
                    src_mod, leaf = _resolve(main, attr)
                    dst_mod, _ = _resolve(tm.module, attr)
                    setattr(dst_mod, leaf, getattr(src_mod, leaf))
            self.tied_modules_by_layer_index[i] = tm

    # ---- queries
    @property
    def tied_information_by_key(self) -> dict[str, TieRecord]:
        return self.records

    def get_module_by_layer_index(self, layer_index: int) -> torch.nn.Module:
        return self.tied_modules_by_layer_index[layer_index].module

    def get_tied_weight_attributes_by_layer_index(self, layer_index: int) -> set[str]:
        return self.tied_modules_by_layer_index[layer_index].tied_weight_attributes

    def local_parameters_and_process_groups(self) -> list[tuple[torch.nn.Parameter, Any, set[int]]]:
        out = []
        for key in sorted(self.tied_parameters_by_key):
            rec = self.records[key]
            for name in sorted(self.tied_parameters_by_key[key]):
                if len(rec.pipe_parallel_ranks) > 1 and dist.is_initialized():
                    assert rec.process_group is not None
                out.append((self.tied_parameters_by_key[key][name], rec.process_group, rec.pipe_parallel_ranks))
        return out

    def layer_index_is_tied_global_duplicate(self, layer_index: int) -> bool:
        tm = self.tied_modules_by_layer_index.get(layer_index)
        return tm is not None and not tm.is_main

    def layer_index_is_tied_local_duplicate(self, layer_index: int) -> bool:
        tm = self.tied_modules_by_layer_index.get(layer_index)
        return tm is not None and not tm.is_local_main

    def layer_index_to_tied_local_duplicate_parameter_names(self, layer_index: int) -> set[str]:
        tm = self.tied_modules_by_layer_index.get(layer_index)
        if tm is None or tm.is_local_main:
            return set()
        return tm.tied_weight_attributes
