"""Embedding table sharded over the vocabulary.

Each tensor-parallel rank owns rows ``[rank * V/mp, (rank + 1) * V/mp)``; ids outside the shard
produce zero rows and the partial results are summed over the group (all-reduce, or reduce-scatter
over tokens in sequence-parallel mode).  ``finetunable_token_ids`` restricts the gradient to the
listed rows.  Semantics of src/scaling/core/nn/linear/vocab_parallel_embedding.py:23-196; the masked
gather and its deterministic scatter-add backward are one CUDA kernel each.
"""

from __future__ import annotations

from typing import Any, Callable, Optional

import torch

from ....ops import functional as K
from ....parallel.collectives import all_reduce, all_reduce_scatter_to_sequence_parallel
from ....parallel.topology import Topology
from ..parameter_meta import UMUP_WEIGHT_TYPE, CoreParameterMeta, UMuPParameterMeta
from ..scale import scale_bwd, scale_fwd
from ..umup import UMuParametrization
from .parallel_linear import get_device


class VocabParallelEmbedding(torch.nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, finetunable_token_ids: Optional[list[int]] = None,
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.float32,
                 topology: Optional[Topology] = None,
                 init_method: Callable[[torch.Tensor], torch.Tensor] = torch.nn.init.xavier_normal_) -> None:
        super().__init__()
        assert not (topology is not None and device is not None), "cannot specify both device and topology"
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self._device = get_device(topology, device)
        self.dtype = dtype
        self.topology = topology
        self.init_method = init_method
        self.model_parallel_size = 1 if topology is None else topology.config.model_parallel_size
        mp = self.model_parallel_size
        assert num_embeddings % mp == 0, (
            f"cannot parallelize embedding, num_embeddings ({num_embeddings}) needs to be divisible by "
            f"model parallel size ({mp})"
        )
        self.vocab_size_per_partition = num_embeddings // mp
        self.vocab_start_index = 0 if topology is None else topology.model_parallel_rank * self.vocab_size_per_partition
        self.vocab_end_index = self.vocab_start_index + self.vocab_size_per_partition
        self.weight = torch.nn.Parameter(
            torch.empty(self.vocab_size_per_partition, embedding_dim, device=self._device, dtype=dtype)
        )
        init_method(self.weight)
        CoreParameterMeta.register_on_parameter(self.weight, is_model_parallel=True, model_parallel_dimension=0)

        ids = list(finetunable_token_ids or [])
        if ids:
            local = [t - self.vocab_start_index for t in ids if self.vocab_start_index <= t < self.vocab_end_index]
            row_mask = torch.zeros(self.vocab_size_per_partition, 1, device=self._device, dtype=dtype)
            if local:
                row_mask[torch.tensor(local, device=self._device)] = 1
            self.weight.register_hook(lambda g: None if g is None else g * row_mask)

        self._use_umup = False
        self.forward_multiplier = 1.0
        self.weight_grad_multiplier = 1.0

    def umup_setup(self, effective_batch_size: int, depth: int, **kwargs: Any) -> None:
        self._use_umup = True
        meta: CoreParameterMeta = self.weight.core_parameter_meta  # type: ignore[attr-defined]
        meta.umup_meta = UMuPParameterMeta(weight_type=UMUP_WEIGHT_TYPE.INPUT_EMBEDDING, on_residual=False)
        UMuParametrization.apply_umup_to_weight(self.weight, self.model_parallel_size, effective_batch_size, depth)
        self.forward_multiplier = meta.umup_meta.forward_multiplier
        self.weight_grad_multiplier = meta.umup_meta.grad_multiplier

    def forward(self, x: torch.Tensor, scatter_tokens: bool = True) -> torch.Tensor:
        """``scatter_tokens=False`` keeps the full (all-reduced) output under sequence parallelism, for callers that
        edit positions of the sequence before they shard it themselves."""
        w = scale_bwd(self.weight, self.weight_grad_multiplier) if self._use_umup else self.weight
        # ids outside [vocab_start, vocab_end) come back as zero rows
        out = K.embedding(x, w, self.vocab_start_index)
        if self._use_umup:
            out = scale_fwd(out, self.forward_multiplier)
        if self.model_parallel_size > 1:
            assert self.topology is not None
            if self.topology.config.sequence_parallel and scatter_tokens:
                out = all_reduce_scatter_to_sequence_parallel(out, self.topology)
            else:
                out = all_reduce(out, self.topology)
        return out
