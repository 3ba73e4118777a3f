"""Pre-norm transformer block: ``x + attn(norm(x))`` then ``x + mlp(norm(x))``, each followed by an
optional bottleneck adapter; dropout after both sub-blocks uses the tensor-parallel-constant RNG.
Sub-module names (``input_layernorm``, ``self_attention``, ``post_attention_layernorm``, ``mlp``,
``attn_adapter_{name}``, ``mlp_adapter_{name}``) are the checkpoint keys of the reference
(src/scaling/transformer/model/layers/layer.py:45-345)."""

from __future__ import annotations

from functools import partial
from typing import Callable, Optional, Union

import torch

from ....core.nn.attention import ParallelSelfAttention
from ....core.nn.mlp import ParallelMLP, ParallelSwiGLUMLP
from ....core.nn.norm import get_norm
from ....core.nn.residual import NormedResidualAdd, NormedResidualSplit
from ....core.nn.rotary import RotaryConfig
from ....core.nn.umup import UMuParametrization
from ....ops import functional as K
from ....parallel.topology import Topology
from ...context.config import MLPType, TransformerArchitectureConfig
from .base import TransformerLayerBaseIO, TransformerLayerIO, record_embedding
from .embedding import _device


class TransformerLayer(TransformerLayerBaseIO):
    def __init__(self, architecture_config: TransformerArchitectureConfig, layer_index: int,
                 topology: Optional[Topology] = None,
                 init_method: Callable[[torch.Tensor], torch.Tensor] = torch.nn.init.xavier_normal_,
                 device: Optional[torch.device] = None) -> None:
        super().__init__()
        a = architecture_config
        self.architecture_config = a
        self.topology = topology
        self.layer_index = layer_index
        dev = device if device is not None else _device(topology)
        explicit = None if topology is not None else dev
        bitfit = getattr(a.bitfit_bias_config, "name", None)
        dtype = a.precision.dtype
        norm = partial(get_norm, norm_type=a.norm_type, layernorm_config=a.layernorm, dimensions=a.hidden_size,
                       device=dev, dtype=dtype, bitfit_bias_name=bitfit, topology=topology, umup_on_residual=True)
        attn_mult = act_mult = residual_mults = None
        if a.umup.enable:
            attn_mult, act_mult = a.umup.attn_mult, a.umup.act_mult
            residual_mults = UMuParametrization.get_umup_transformer_residual_mults(
                residual_mult=a.umup.residual_mult, residual_attn_ratio=a.umup.residual_attn_ratio,
                num_layers=a.num_layers,
            )
        self.input_layernorm = norm()
        head_dim = a.hidden_size // a.num_attention_heads
        self.self_attention = ParallelSelfAttention(
            hidden_size=a.hidden_size, num_attention_heads=a.num_attention_heads,
            num_local_attention_heads=a.num_local_attention_heads,
            local_attention_window_size=a.local_attention_window_size, masked_softmax_config=a.masked_softmax,
            causal=a.causal, dropout_attention_probs=a.dropout_attention_probs,
            rotary_config=RotaryConfig(dimensions=int(a.rotary_percentage * head_dim),
                                       max_seq_length=a.sequence_length, base=a.rotary_embedding_base),
            relative_position_embedding_type=a.relative_position_embedding_type, bias=a.attention_bias,
            topology=topology, device=explicit, dtype=dtype, bitfit_bias_name=bitfit, init_method=init_method,
            lora_config=a.lora_config, norm_type=a.norm_type, key_query_norm=a.key_query_norm,
            layernorm_config=a.layernorm, qkv_in_one=a.attention_qkv_in_one, num_kv_heads=a.attention_num_kv_heads,
            use_matmul=a.attention_use_matmul, umup_is_first_layer=False, umup_is_last_layer=False,
            umup_on_residual=True, umup_mult=attn_mult, fp8_config=a.fp8_config_attention,
            fp8_config_dense_out=a.fp8_config_attention_dense_out,
        )
        self.dropout_attention = torch.nn.Dropout(a.dropout_after_attention)
        self.dropout_attention.kernel_dropout = True  # applied by the fused dropout + residual kernel on the GPU
        self.attn_residual_split = NormedResidualSplit(residual_mults, 2 * layer_index, True)
        self.attn_residual_add = NormedResidualAdd(residual_mults, 2 * layer_index, True)
        self.post_attention_layernorm = norm()
        if topology is not None and topology.config.sequence_parallel and topology.config.model_parallel_size > 1:
            # attention and MLP take this rank's tokens and gather them inside their first GEMMs
            self.input_layernorm.defer_gather = True
            self.post_attention_layernorm.defer_gather = True
        mlp_cls = {MLPType.DEFAULT: ParallelMLP, MLPType.SWIGLU: ParallelSwiGLUMLP}[a.mlp_type]
        self.mlp: Union[ParallelMLP, ParallelSwiGLUMLP] = mlp_cls(
            io_features=a.hidden_size, intermediate_feature_factor=a.mlp_factor, bias=a.mlp_bias, topology=topology,
            device=explicit, dtype=dtype, bitfit_bias_name=bitfit, init_method=init_method,
            umup_is_first_layer=False, umup_is_last_layer=False, umup_on_residual=True, umup_mult=act_mult,
            fp8_config=a.fp8_config_mlp, fp8_config_dense_out=a.fp8_config_mlp_dense_out,
        )
        self.dropout_mlp = torch.nn.Dropout(a.dropout_after_mlp)
        self.dropout_mlp.kernel_dropout = True
        self.mlp_residual_split = NormedResidualSplit(residual_mults, 2 * layer_index + 1, True)
        self.mlp_residual_add = NormedResidualAdd(residual_mults, 2 * layer_index + 1, True)
        if a.adapter_config is not None:
            self.load_adapter(explicit)

    def load_adapter(self, device: Optional[torch.device] = None) -> None:
        a = self.architecture_config
        cfg = a.adapter_config
        assert cfg is not None
        make = partial(ParallelMLP, io_features=a.hidden_size, bias=False, topology=self.topology, device=device,
                       dtype=a.precision.dtype, init_method=partial(torch.nn.init.normal_, mean=0.0, std=cfg.init_std))
        if cfg.attention_downsampling_factor is not None:
            self.attn_adapter_name = f"attn_adapter_{cfg.name}"
            setattr(self, self.attn_adapter_name, make(intermediate_feature_factor=cfg.attention_downsampling_factor))
        if cfg.mlp_downsampling_factor is not None:
            self.mlp_adapter_name = f"mlp_adapter_{cfg.name}"
            setattr(self, self.mlp_adapter_name, make(intermediate_feature_factor=cfg.mlp_downsampling_factor))

    def apply_adapter(self, x: torch.Tensor, adapter_name: str) -> torch.Tensor:
        assert hasattr(self, adapter_name), f"cannot use adapter '{adapter_name}' as it is not initialized"
        t = self.topology
        if t is not None and t.config.sequence_parallel and t.config.model_parallel_size > 1:
            # the residual stream holds this rank's tokens: the adapter's first linear gathers them, its last one
            # scatters the result again
            from ....parallel.collectives import SequenceShard

            x = SequenceShard(x, t)  # type: ignore[assignment]
        return getattr(self, adapter_name)(x)

    def _dropout(self, module: torch.nn.Dropout, x: torch.Tensor) -> torch.Tensor:
        if module.p == 0.0 or not self.training:
            return x
        if self.topology is not None and self.topology.has_model_parallel_constant_rng:
            with self.topology.model_parallel_constant_rng():
                return module(x)
        return module(x)

    def _dropout_residual(self, dropout: torch.nn.Dropout, add: NormedResidualAdd, branch: torch.Tensor,
                          skip: torch.Tensor) -> torch.Tensor:
        """``dropout(branch) + skip`` (with the u-muP scales of ``add``) as one kernel on the GPU: the mask comes from
        the topology's counter-based stream, identical on all tensor-parallel ranks and recomputed in the backward
        pass; token shards (sequence parallelism) take disjoint parts of it."""
        t = self.topology
        if not (branch.is_cuda and t is not None and branch.shape == skip.shape and branch.dtype == skip.dtype):
            return add(self._dropout(dropout, branch), skip)
        p = dropout.p if self.training else 0.0
        xs, rs = (add.residual_scale, add.skip_scale) if add._use_umup else (1.0, 1.0)
        sharded = t.config.sequence_parallel and t.config.model_parallel_size > 1
        offset = t.model_parallel_rank * ((branch.numel() + 3) // 4 * 4) if sharded else 0
        return K.dropout_add(branch, skip, p, t.kernel_rng, True, xs, rs, offset, scale_grad=not add._use_umup)

    def attention_block(self, hidden_state: torch.Tensor, cumulative_seq_lengths: torch.Tensor,
                        position_ids: torch.Tensor, use_cache: bool = False, reset_cache: bool = False,
                        cache_index: int = 0, attention_scores_manipulation: Optional[torch.Tensor] = None,
                        attentions_score_manipulation_log_additive: Union[bool, list[bool]] = True,
                        doc_ranges: Optional[tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
        branch, skip = self.attn_residual_split(hidden_state)
        branch = self.self_attention(
            self.input_layernorm(branch), cumulative_seq_lengths=cumulative_seq_lengths, position_ids=position_ids,
            use_cache=use_cache, reset_cache=reset_cache, cache_index=cache_index,
            attention_scores_manipulation=attention_scores_manipulation,
            attentions_score_manipulation_log_additive=attentions_score_manipulation_log_additive,
            doc_ranges=doc_ranges,
        )
        h = self._dropout_residual(self.dropout_attention, self.attn_residual_add, branch, skip)
        if hasattr(self, "attn_adapter_name"):
            h = h + self.apply_adapter(h, self.attn_adapter_name)
        return h

    def mlp_block(self, hidden_state: torch.Tensor) -> torch.Tensor:
        branch, skip = self.mlp_residual_split(hidden_state)
        branch = self.mlp(self.post_attention_layernorm(branch))
        h = self._dropout_residual(self.dropout_mlp, self.mlp_residual_add, branch, skip)
        if hasattr(self, "mlp_adapter_name"):
            h = h + self.apply_adapter(h, self.mlp_adapter_name)
        return h

    def forward(self, x: TransformerLayerIO) -> TransformerLayerIO:
        s = x.inference_settings
        assert x.cumulative_seq_lengths is not None or x.cumulative_seq_lengths_padded is not None
        h = self.attention_block(
            x.activations, cumulative_seq_lengths=x.cumulative_seq_lengths, position_ids=x.position_ids,
            use_cache=s.use_cache if s else False, reset_cache=s.reset_cache if s else False,
            cache_index=s.cache_index if s else 0, attention_scores_manipulation=x.attention_scores_manipulation,
            attentions_score_manipulation_log_additive=s.control_log_additive_batch if s else True,
            doc_ranges=x.document_ranges(),
        )
        h = self.mlp_block(h)
        record_embedding(x, self.layer_index + 1, h)
        return x.evolve(activations=h, embeddings_head=None)
