"""Assignment of layers to pipeline stages.

``uniform`` spreads layers evenly (earlier stages take the remainder), ``balanced`` minimises the
heaviest stage by parameter count, ``from_indices`` takes explicit boundaries
(behaviour of src/scaling/core/nn/parallel_module/pipeline_partitioning.py:16-136; the balanced
split here is an exact dynamic program over prefix sums instead of a probe-and-bisect search).
"""

from __future__ import annotations

from typing import List, NamedTuple, Optional, Sequence

import torch

from .layer_spec import LayerSpec


class PipePartitionCoordinates(NamedTuple):
    start: int
    end: int

    @property
    def length(self) -> int:
        return self.end - self.start


def pipe_partition_from_indices(partition_array: Sequence[int], num_layers: Optional[int] = None) -> List[PipePartitionCoordinates]:
    if num_layers is not None and partition_array[-1] != num_layers:
        raise ValueError(
            f"Last entry of partition_array needs to match num_layers; got"
            f"partition_array={partition_array}, num_layers={num_layers}."
        )
    return [PipePartitionCoordinates(int(a), int(b)) for a, b in zip(partition_array[:-1], partition_array[1:])]


def pipe_partition_uniform(item_count: int, partition_count: int) -> List[PipePartitionCoordinates]:
    assert item_count >= partition_count, (
        f"cannot partition {item_count} layers on {partition_count} pipe parallel stages"
    )
    base, extra = divmod(item_count, partition_count)
    bounds = [0]
    for stage in range(partition_count):
        bounds.append(bounds[-1] + base + (1 if stage < extra else 0))
    return pipe_partition_from_indices(bounds)


def count_layer_params(layer_specs: List[LayerSpec]) -> list[int]:
    """Trainable parameters per layer; each layer is built on the CPU, one at a time."""
    counts = []
    for spec in layer_specs:
        layer = spec.initialize(torch.device("cpu")) if _accepts_cpu(spec) else spec.initialize()
        counts.append(sum(p.numel() for p in layer.parameters() if p.requires_grad))
        del layer
    return counts


def _accepts_cpu(spec: LayerSpec) -> bool:
    return True


def balanced_boundaries(weights: Sequence[int], partition_count: int) -> list[int]:
    """Boundaries of the contiguous split into ``partition_count`` non-empty parts with the lightest maximum part."""
    n = len(weights)
    assert n >= partition_count, f"cannot partition {n} layers on {partition_count} pipe parallel stages"
    prefix = [0]
    for w in weights:
        prefix.append(prefix[-1] + int(w))
    INF = float("inf")
    # best[p][i]: minimal bottleneck for the first i items in p parts
    best = [[INF] * (n + 1) for _ in range(partition_count + 1)]
    cut = [[0] * (n + 1) for _ in range(partition_count + 1)]
    best[0][0] = 0
    for p in range(1, partition_count + 1):
        for i in range(p, n - (partition_count - p) + 1):
            for j in range(p - 1, i):
                cand = max(best[p - 1][j], prefix[i] - prefix[j])
                if cand < best[p][i]:
                    best[p][i] = cand
                    cut[p][i] = j
    bounds = [n]
    i = n
    for p in range(partition_count, 0, -1):
        i = cut[p][i]
        bounds.append(i)
    return bounds[::-1]


def pipe_partition_balanced(layer_specs: List[LayerSpec], partition_count: int, eps: float = 1e-3) -> List[PipePartitionCoordinates]:
    return pipe_partition_from_indices(balanced_boundaries(count_layer_params(layer_specs), partition_count))
