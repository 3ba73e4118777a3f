"""Final norm and output heads.

``LayerNormWrapper`` applies the last norm.  ``TransformerLMHead`` is a column-parallel projection to
the vocabulary; ``TransformerLMHeadTied`` multiplies with the (shared) embedding matrix.  While
training with tensor parallelism both return logits *sharded over the vocabulary* and the
cross-entropy loss works on the shards directly, so the ``[tokens, vocab]`` matrix is never gathered;
for inference (no topology) and on request (``gather_logits``) they return full logits like the
reference (src/scaling/transformer/model/layers/lm_head.py:16-68, lm_head_tied.py:16-53).
``TransformerEmbeddingHead`` pools token states into one embedding per sequence
(embedding_head.py:11-118).
"""

from __future__ import annotations

from typing import Callable, Optional

import torch

from ....core.nn.linear import ColumnParallelLinear, VocabParallelEmbedding
from ....core.nn.norm import get_norm
from ....core.nn.parameter_meta import UMUP_WEIGHT_TYPE
from ....core.nn.scale import scale_bwd
from ....ops import functional as K
from ....parallel.collectives import all_concat, copy_to_tensor_model_parallel_region
from ....parallel.topology import Topology
from ...context.config import PoolingMethod, TransformerArchitectureConfig
from .base import TransformerLayerBaseIO, TransformerLayerIO, record_embedding
from .embedding import _device


class LayerNormWrapper(TransformerLayerBaseIO):
    def __init__(self, architecture_config: TransformerArchitectureConfig, layer_index: int,
                 topology: Optional[Topology] = None, umup_on_residual: Optional[bool] = None,
                 device: Optional[torch.device] = None):
        super().__init__()
        a = architecture_config
        self.topology = topology
        self.architecture_config = a
        self.layer_index = layer_index
        self.norm = get_norm(
            norm_type=a.norm_type, layernorm_config=a.layernorm, dimensions=a.hidden_size,
            device=device if device is not None else _device(topology), dtype=a.precision.dtype,
            bitfit_bias_name=getattr(a.bitfit_bias_config, "name", None), topology=topology,
            umup_on_residual=umup_on_residual,
        )

    def forward(self, x: TransformerLayerIO) -> TransformerLayerIO:
        h = self.norm(x.activations)
        record_embedding(x, self.layer_index + 1, h)
        return x.evolve(activations=h, attention_scores_manipulation=None, embeddings_head=None)


def _finetunable_row_mask(weight: torch.Tensor, token_ids: list[int], vocab_start: int) -> Optional[torch.Tensor]:
    if not token_ids:
        return None
    rows = weight.shape[0]
    mask = torch.zeros(rows, 1, device=weight.device, dtype=weight.dtype)
    local = [t - vocab_start for t in token_ids if vocab_start <= t < vocab_start + rows]
    if local:
        mask[torch.tensor(local, device=weight.device)] = 1
    return mask


class _LMHeadBase(TransformerLayerBaseIO):
    gather_logits: bool = False  # set True to always return full-vocabulary logits under tensor parallelism

    def _finish(self, x: TransformerLayerIO, logits: torch.Tensor) -> TransformerLayerIO:
        t = self.topology
        if t is not None and t.config.model_parallel_size > 1 and (self.gather_logits or not self.training):
            logits = all_concat(logits, t)
        if self.training and logits.grad_fn is not None:
            # Nothing but the loss reads the logits of a training step: the loss may write their gradient over them.
            logits._sb200_loss_may_overwrite = True  # type: ignore[attr-defined]
        return x.evolve(activations=logits, attention_scores_manipulation=None, embeddings_head=None)


class TransformerLMHead(_LMHeadBase):
    def __init__(self, architecture_config: TransformerArchitectureConfig,
                 init_method: Callable[[torch.Tensor], torch.Tensor] = torch.nn.init.xavier_normal_,
                 topology: Optional[Topology] = None, device: Optional[torch.device] = None):
        super().__init__()
        a = architecture_config
        self.topology = topology
        self.linear = ColumnParallelLinear(
            in_features=a.hidden_size, out_features=a.vocab_size, bias=False, topology=topology,
            device=None if topology is not None else (device or _device(None)), dtype=a.precision.dtype,
            init_method=init_method, parallel_output=True, umup_weight_type=UMUP_WEIGHT_TYPE.OUTPUT_WEIGHT,
            umup_on_residual=False, fp8_config=a.fp8_config_lm_head,
        )
        mp_rank = 0 if topology is None else topology.model_parallel_rank
        mask = _finetunable_row_mask(self.linear.weight, list(a.finetunable_token_ids),
                                     mp_rank * self.linear.weight.shape[0])
        if mask is not None:
            self.linear.weight.register_hook(lambda g: None if g is None else g * mask)

    def forward(self, x: TransformerLayerIO) -> TransformerLayerIO:
        return self._finish(x, self.linear(x.activations))


class TransformerLMHeadTied(_LMHeadBase):
    def __init__(self, architecture_config: TransformerArchitectureConfig,
                 init_method: Callable[[torch.Tensor], torch.Tensor] = torch.nn.init.xavier_normal_,
                 topology: Optional[Topology] = None, device: Optional[torch.device] = None):
        super().__init__()
        a = architecture_config
        self.topology = topology
        self.embedding = VocabParallelEmbedding(
            num_embeddings=a.vocab_size, embedding_dim=a.hidden_size, topology=topology,
            device=None if topology is not None else (device or _device(None)), dtype=a.precision.dtype,
            init_method=init_method, finetunable_token_ids=a.finetunable_token_ids,
        )

    def forward(self, x: TransformerLayerIO) -> TransformerLayerIO:
        h = x.activations
        t = self.topology
        if t is not None and t.config.model_parallel_size > 1 and not t.config.sequence_parallel:
            h = copy_to_tensor_model_parallel_region(h, t)
        return self._finish(x, K.linear(h, self.embedding.weight))


class TransformerEmbeddingHead(TransformerLayerBaseIO):
    def __init__(self, architecture_config: TransformerArchitectureConfig, topology: Optional[Topology] = None,
                 device: Optional[torch.device] = None):
        super().__init__()
        cfg = architecture_config.embedding_head_config
        assert cfg is not None, "Initializing EmbeddingHead without embedding_head_config is not possible"
        self.embedding_head_config = cfg
        self.topology = topology
        dev = device if device is not None else _device(topology)
        width = architecture_config.hidden_size
        for i, out in enumerate(cfg.proj_layers or []):
            setattr(self, f"embedding_head_proj_{cfg.name}_{i}",
                    torch.nn.Linear(width, out, bias=False, device=dev, dtype=architecture_config.precision.dtype))
            width = out

    def apply_embedding_head_proj(self, hidden_states: torch.Tensor) -> torch.Tensor:
        cfg = self.embedding_head_config
        for i, _ in enumerate(cfg.proj_layers or []):
            if i > 0:
                hidden_states = torch.nn.functional.gelu(hidden_states)
            hidden_states = getattr(self, f"embedding_head_proj_{cfg.name}_{i}")(hidden_states)
        return hidden_states

    @staticmethod
    def apply_last_token_pooling(embeddings: torch.Tensor, loss_weights: torch.Tensor) -> torch.Tensor:
        n = loss_weights.size(1)
        last = (n - 1 - torch.argmax(torch.flip(loss_weights, dims=(1,)), dim=1)).clamp(min=0)
        masked = embeddings * loss_weights.unsqueeze(-1).float()
        return masked[torch.arange(embeddings.shape[0], device=embeddings.device), last]

    @staticmethod
    def apply_mean_pooling(embeddings: torch.Tensor, loss_weights: torch.Tensor, weighted: bool = False) -> torch.Tensor:
        in_dtype = embeddings.dtype
        e = embeddings.float()
        w = loss_weights.unsqueeze(-1).float()
        position_weight = loss_weights.float().cumsum(dim=1).unsqueeze(-1) if weighted else w
        num = (e * w * position_weight).sum(dim=1)
        den = (w * position_weight).sum(dim=1)
        if float(den.sum()) == 0.0:
            return torch.zeros_like(num).to(in_dtype)
        return (num / den).to(in_dtype)

    def apply_pooling(self, hidden_states: torch.Tensor, loss_weights: torch.Tensor,
                      pooling_method: PoolingMethod) -> torch.Tensor:
        if pooling_method == PoolingMethod.WEIGHTED_MEAN:
            return self.apply_mean_pooling(hidden_states, loss_weights, weighted=True)
        if pooling_method == PoolingMethod.MEAN:
            return self.apply_mean_pooling(hidden_states, loss_weights)
        if pooling_method == PoolingMethod.LAST_TOKEN:
            return self.apply_last_token_pooling(hidden_states, loss_weights)
        raise NotImplementedError(pooling_method)

    def forward(self, x: TransformerLayerIO) -> TransformerLayerIO:
        assert x.loss_weights is not None, "loss_weights are required for embedding pooling"
        acts = x.activations
        t = self.topology
        if t is not None and t.config.sequence_parallel and t.config.model_parallel_size > 1:
            # This head is replicated: every tensor-parallel rank computes the same loss from the gathered sequence
            # and sends the same, complete gradient back into the gather, whose backward pass sums over the ranks.
            acts = scale_bwd(acts, 1.0 / t.config.model_parallel_size)
        h = self.apply_embedding_head_proj(acts) if self.embedding_head_config.proj_layers else acts
        pooled = self.apply_pooling(h.float(), x.loss_weights, self.embedding_head_config.pooling)
        return TransformerLayerIO(
            activations=pooled, position_ids=x.position_ids, cumulative_seq_lengths=x.cumulative_seq_lengths,
            cumulative_seq_lengths_padded=x.cumulative_seq_lengths_padded, loss_weights=x.loss_weights,
        )
