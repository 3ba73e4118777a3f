"""Input layer: vocab-parallel token embedding, dropout, optional image-prefix / soft-prompt splice,
and the attention-manipulation ("AtMan") matrix for controlled inference.

Behaviour follows src/scaling/transformer/model/layers/embedding.py:29-375.  The embedding dropout
uses the tensor-parallel-constant RNG stream so that all ranks of a TP group drop the same elements.
"""

from __future__ import annotations

import math
from typing import Any, Callable, Optional

import torch

from ....core.nn.linear import VocabParallelEmbedding
from ....core.nn.parallel_module import BaseLayer
from ....ops import functional as K
from ....parallel.topology import Topology
from ...context.config import TransformerArchitectureConfig
from ...data.text_dataset_batch import TextDatasetBatch
from .base import TransformerLayerIO, record_embedding


def _device(topology: Optional[Topology]) -> torch.device:
    if topology is not None:
        return topology.device
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def control_factor_from_cosine_similarity(control_factor: float, cosine_similarity: float) -> float:
    """Interpolate between no control (similarity 0) and the full factor (similarity 1)."""
    if 0.0 <= cosine_similarity <= 1.0:
        return (1.0 - control_factor) * (1.0 - cosine_similarity) + control_factor
    return 1.0


def cosine_similarity_matrix(embeddings: torch.Tensor, eps: float = 1e-8) -> torch.Tensor:
    """``[b, s, s]`` cosine similarities between all token embeddings of each batch item (fp32, clipped)."""
    e = embeddings.detach().float()
    e = e / e.norm(dim=-1, keepdim=True).clamp_min(eps)
    return torch.matmul(e, e.transpose(1, 2)).clip(-1, 1).cpu()


class BaseEmbeddingInput(BaseLayer[TextDatasetBatch, TransformerLayerIO, TransformerLayerIO]):
    def __init__(self, architecture_config: TransformerArchitectureConfig, topology: Optional[Topology] = None,
                 init_method: Callable[[torch.Tensor], torch.Tensor] = torch.nn.init.xavier_normal_,
                 device: Optional[torch.device] = None):
        super().__init__()
        self.architecture_config = architecture_config
        self.topology = topology
        dev = device if device is not None else _device(topology)
        self.embedding = VocabParallelEmbedding(
            num_embeddings=architecture_config.vocab_size, embedding_dim=architecture_config.hidden_size,
            topology=topology, device=None if topology is not None else dev,
            dtype=architecture_config.precision.dtype, init_method=init_method,
            finetunable_token_ids=architecture_config.finetunable_token_ids,
        )
        self.dropout = torch.nn.Dropout(p=architecture_config.dropout_embedding)
        self.dropout.kernel_dropout = True  # applied by the dropout kernel on the GPU
        if architecture_config.image_encoder:
            from ..image_encoder import ImageEncoder

            self.image_encoder = ImageEncoder(
                out_features=architecture_config.hidden_size, dropout_p=architecture_config.dropout_image_encoder,
                layernorm_config=architecture_config.layernorm, dtype=architecture_config.precision.dtype, device=dev,
            )
        self.softprompt_name: Optional[str] = None
        if architecture_config.softprompt_config is not None:
            sp = architecture_config.softprompt_config
            self.softprompt_name = sp.name
            p = torch.nn.Parameter(torch.zeros((sp.n_tokens, architecture_config.hidden_size),
                                               dtype=architecture_config.precision.dtype, device=dev))
            init_method(p)
            setattr(self, f"softprompt_{sp.name}", p)
        self.cache: dict[int, Optional[torch.Tensor]] = {}

    def _dropout(self, fn: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor) -> torch.Tensor:
        if self.topology is not None and self.topology.has_model_parallel_constant_rng:
            with self.topology.model_parallel_constant_rng():
                return fn(x)
        return fn(x)

    def forward(self, x: TextDatasetBatch) -> TransformerLayerIO:
        s = x.inference_settings
        use_cache, reset_cache, cache_index = (s.use_cache, s.reset_cache, s.cache_index) if s else (False, False, 0)
        if reset_cache:
            self.cache[cache_index] = None
        assert x.input_token_ids is not None
        t = self.topology
        sequence_parallel = t is not None and t.config.sequence_parallel and t.config.model_parallel_size > 1
        # image and soft-prompt positions are written into the whole sequence: under sequence parallelism the
        # embedding then stays replicated until they are in, and is split over the ranks afterwards
        splice_full = sequence_parallel and (x.input_images is not None or self.softprompt_name is not None)
        h = self.embedding(x.input_token_ids, scatter_tokens=not splice_full)
        if self.dropout.p > 0.0 and self.training:
            if h.is_cuda and t is not None:  # counter-based mask from the topology's stream, one kernel
                sharded = sequence_parallel and not splice_full
                offset = t.model_parallel_rank * ((h.numel() + 3) // 4 * 4) if sharded else 0
                h = K.dropout_add(h, None, self.dropout.p, t.kernel_rng, True, elem_offset=offset)
            else:
                h = self._dropout(self.dropout, h)

        if x.input_images is not None:
            img = self._dropout(self.image_encoder, x.input_images)
            locations = x.input_image_locations
            if locations is None and not self.training:
                assert s is not None and s.input_image_locations is not None
                locations = s.input_image_locations
            if locations is not None:
                assert len(locations) == img.shape[0]
                h = h.clone()
                for emb, (b, start, end) in zip(img, locations):
                    h[int(b), int(start):int(end)] = emb
            else:  # pre-training: the image tokens lead the sequence; concatenation keeps gradients
                h = torch.cat([img, h[:, img.shape[1]:, :]], dim=1).contiguous()

        if self.softprompt_name is not None:
            sp = getattr(self, f"softprompt_{self.softprompt_name}")
            h = torch.cat([sp.unsqueeze(0).expand(h.shape[0], -1, -1), h[:, sp.shape[0]:, :]], dim=1).contiguous()

        if splice_full:
            from ....parallel.collectives import shard_to_sequence_parallel_region

            h = shard_to_sequence_parallel_region(h, t)

        out = TransformerLayerIO(
            activations=h, position_ids=x.position_ids, cumulative_seq_lengths=x.cumulative_seq_lengths,
            cumulative_seq_lengths_padded=x.cumulative_seq_lengths_padded, loss_weights=x.loss_weights,
            inference_settings=s, embeddings=x.embeddings,
        )
        record_embedding(out, 0, h)
        if s is not None and s.inference_control_parameters is not None:
            out.attention_scores_manipulation = self._attention_manipulation(h, out, use_cache, reset_cache, cache_index)
        return out

    def _attention_manipulation(self, h: torch.Tensor, io: TransformerLayerIO, use_cache: bool, reset_cache: bool,
                                cache_index: int) -> torch.Tensor:
        """``[b, 1, s, s]`` matrix added to (log-additive) or multiplied with the attention scores."""
        s = io.inference_settings
        params = s.inference_control_parameters  # type: ignore[union-attr]
        b, n = h.shape[0], h.shape[1]
        assert len(params) == b, "number of inference_control_parameters does not match batch size"
        m = torch.zeros(b, 1, n, n, device=h.device, dtype=h.dtype)
        for i, p in enumerate(params):
            if not p.control_log_additive:
                m[i] = 1.0
        sim = None
        if any(p.contextual_control_threshold is not None for p in params):
            basis = h
            if use_cache:
                if not reset_cache and self.cache.get(cache_index) is not None:
                    basis = torch.cat([self.cache[cache_index], basis], dim=1)  # type: ignore[list-item]
                self.cache[cache_index] = basis
            sim = cosine_similarity_matrix(basis)
        for i, p in enumerate(params):
            if p is None or p.controls is None or all(c.token_index == -1 for c in p.controls):
                continue
            factors: dict[int, float] = {}
            for c in p.controls:
                if c.token_index < 0:
                    continue
                factors[c.token_index] = c.factor
                if p.contextual_control_threshold is not None:
                    assert sim is not None
                    row = sim[i][c.token_index]
                    for j in (row >= p.contextual_control_threshold).nonzero().view(-1).tolist():
                        if j == c.token_index:
                            continue
                        f = control_factor_from_cosine_similarity(c.factor, float(row[j]))
                        factors[j] = min(f, factors.get(j, 0.0))
            for j, f in factors.items():
                if reset_cache and io.loss_weights is not None:  # weights are set on the first pass only
                    io.loss_weights[i, j] = io.loss_weights[i, j] * f
                if p.control_log_additive:
                    m[i, :, :, j] = -10000.0 if f == 0.0 else math.log(f)
                else:
                    m[i, :, :, j] = f
        return m

    @staticmethod
    def input_to_tuple(input: TextDatasetBatch) -> tuple[Any, ...]:
        return input.as_tuple()

    @staticmethod
    def tuple_to_input(d: tuple[Any, ...]) -> TextDatasetBatch:
        return TextDatasetBatch.from_tuple(d)

    @staticmethod
    def output_to_tuple(output: TransformerLayerIO) -> tuple[Any, ...]:
        return output.as_tuple()

    @staticmethod
    def tuple_to_last_stage_activation(d: tuple[Any, ...]) -> TransformerLayerIO:
        return TransformerLayerIO.from_tuple(d)


class EmbeddingInput(BaseEmbeddingInput):
    pass
