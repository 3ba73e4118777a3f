"""Tensor-parallel multi-head self-attention (MHA / GQA / MQA) with packed sequences.

Public surface and parameter names follow the reference's ``ParallelSelfAttention``
(src/scaling/core/nn/attention/attention.py:509-1062): fused ``query_key_value`` (per head
interleaved ``[q_h | k_h | v_h]``) or separate ``query`` / ``key`` / ``value`` projections (needed
for fewer KV heads), optional per-head query/key norm, rotary embeddings with position ids, KV
cache for incremental decoding, LoRA adapters, row-parallel ``dense`` and the sequence-parallel
reduce-scatter.  Internally activations stay token-major (``[batch * seq, heads, head_dim]``),
which is the layout of the packed-sequence attention kernel, so no transposes are needed between
the projections, the rotary kernel and attention.  KV heads fewer than the tensor-parallel width
(MQA under TP) are replicated per rank instead of failing as the reference does.
"""

from __future__ import annotations

from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

import torch

from ....ops import functional as K
from ....ops.attention import attention_mask_from_cu_seqlens, flash_attention
from ....parallel.collectives import (SequenceShard, all_concat, all_reduce_scatter_to_sequence_parallel, all_shard,
                                       copy_to_tensor_model_parallel_region, shard_to_sequence_parallel_region)
from ....parallel.topology import Topology
from ..linear import ColumnParallelLinear, RowParallelLinear, get_device
from ..lora import LoRaConfig, LoRAModuleType, ParallelLoRa
from ..masked_softmax import MaskedSoftmax, MaskedSoftmaxConfig, MaskedSoftmaxKernel
from ..norm import LayerNorm, LayerNormConfig, NormType, RMSNorm, get_norm
from ..parameter_meta import UMUP_WEIGHT_TYPE
from ..rotary import RotaryConfig, RotaryEmbedding, RotaryEmbeddingComplex, apply_rotary_tokens
from ..scale import scale_bwd, scale_fwd
from ..umup import UMuParametrization


class RelativePositionEmbeddingType(Enum):
    NONE = "none"
    ROTARY = "rotary"
    ROTARY_COMPLEX = "rotary_complex"


def get_max_seq_length(cumulative_seq_lengths: torch.Tensor) -> int:
    return int((cumulative_seq_lengths[1:] - cumulative_seq_lengths[:-1]).max().item())


def cumulative_seq_lengths_to_dense_attention_mask(cumulative_seq_lengths: torch.Tensor,
                                                   seq_length_per_batch_item: int, causal: bool) -> torch.Tensor:
    """``[b, 1, s, s]`` boolean mask, True = masked out, from flat cumulative lengths over ``b * s`` tokens."""
    total = int(cumulative_seq_lengths[-1].item())
    allowed = attention_mask_from_cu_seqlens(cumulative_seq_lengths, cumulative_seq_lengths, total, total, causal, None)
    s = seq_length_per_batch_item
    b = total // s
    blocks = torch.stack([allowed[i * s:(i + 1) * s, i * s:(i + 1) * s] for i in range(b)])
    return ~blocks.unsqueeze(1)


class _AttentionCore(torch.nn.Module):
    """Scale bookkeeping shared by the dense and the fused attention kernels (incl. u-muP)."""

    def __init__(self, head_dim: int, dropout_p: float, causal: bool, umup_mult: Optional[float]):
        super().__init__()
        self.head_dim = head_dim
        self.dropout_p = dropout_p
        self.causal = causal
        self.query_key_scaling_factor = 1.0 / (head_dim ** 0.5)
        self.umup_mult = umup_mult
        self.output_scale_factor = 1.0
        self._use_umup = False

    def umup_setup(self, avg_sequence_length: int, **kwargs: Any) -> None:
        assert self.umup_mult is not None
        assert self.causal, "umup currently only implemented for causal attention"
        self._use_umup = True
        self.query_key_scaling_factor, self.output_scale_factor = UMuParametrization.get_umup_attention_scales(
            head_dim=self.head_dim, sequence_length=avg_sequence_length, mult=self.umup_mult, dropout_p=self.dropout_p
        )

    def _pre(self, *ts: torch.Tensor):
        if not self._use_umup:
            return ts
        return tuple(scale_bwd(t, self.output_scale_factor) for t in ts)

    def _post(self, out: torch.Tensor) -> torch.Tensor:
        return scale_fwd(out, self.output_scale_factor) if self._use_umup else out


class ScaledDotProductAttention(_AttentionCore):
    """Dense path: scores ``[b, heads, s, s]`` are materialised; supports attention-score manipulation."""

    def __init__(self, head_dim: int, dropout_p: float, masked_softmax_config: MaskedSoftmaxConfig, causal: bool,
                 use_matmul: bool = False, umup_mult: Optional[float] = None):
        super().__init__(head_dim, dropout_p, causal, umup_mult)
        self.softmax_fn = MaskedSoftmax(masked_softmax_config)
        self.dropout_fn = torch.nn.Dropout(p=dropout_p)
        self.masked_softmax_config = masked_softmax_config
        self.use_matmul = use_matmul

    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                cumulative_seq_lengths: torch.Tensor, attention_scores_manipulation: Optional[torch.Tensor] = None,
                attentions_score_manipulation_log_additive: Union[bool, List[bool]] = True,
                key_offset: int = 0) -> torch.Tensor:
        """query ``[b, sq, h, d]``, key/value ``[b, sk, h, d]`` -> ``[b, sq, h, d]``."""
        query, key, value = self._pre(query, key, value)
        b, sq = query.shape[0], query.shape[1]
        sk = key.shape[1]
        q = query.permute(0, 2, 1, 3)
        k = key.permute(0, 2, 3, 1)
        scores = torch.matmul(q, k) * self.query_key_scaling_factor  # [b, h, sq, sk]
        if sq == sk:
            mask = cumulative_seq_lengths_to_dense_attention_mask(cumulative_seq_lengths, sq, self.causal)
        else:  # incremental decoding against cached keys
            qpos = torch.arange(sq, device=q.device)[:, None] + (sk - sq)
            kpos = torch.arange(sk, device=q.device)[None, :]
            mask = (kpos > qpos if self.causal else torch.zeros(sq, sk, dtype=torch.bool, device=q.device))
            mask = mask[None, None].expand(b, 1, sq, sk)
        if attention_scores_manipulation is not None:
            scores = _manipulate_scores(scores, mask, attention_scores_manipulation,
                                        attentions_score_manipulation_log_additive)
        probs = self.softmax_fn(scores, mask)
        probs = self.dropout_fn(probs)
        out = torch.matmul(probs.to(value.dtype), value.permute(0, 2, 1, 3))  # [b, h, sq, d]
        return self._post(out.permute(0, 2, 1, 3))


def _manipulate_scores(scores: torch.Tensor, mask: torch.Tensor, manipulation: torch.Tensor,
                       log_additive: Union[bool, List[bool]]) -> torch.Tensor:
    """Additive (log space) or multiplicative (after shifting the row minimum to 0) score control."""

    def multiplicative(sc: torch.Tensor, m: torch.Tensor, man: torch.Tensor) -> torch.Tensor:
        floor = sc.masked_fill(m, 10000.0).min(-1).values.unsqueeze(-1)
        return (sc - floor) * man

    if isinstance(log_additive, bool):
        return scores + manipulation if log_additive else multiplicative(scores, mask, manipulation)
    assert len(log_additive) == scores.shape[0]
    rows = []
    for i, additive in enumerate(log_additive):
        rows.append(scores[i] + manipulation[i] if additive else multiplicative(scores[i], mask[i], manipulation[i]))
    return torch.stack(rows)


class FlashAttention(_AttentionCore):
    """Fused path on packed tokens: the score matrix never materialises."""

    def __init__(self, head_dim: int, dropout_p: float, masked_softmax_config: MaskedSoftmaxConfig,
                 num_local_attention_heads: int, causal: bool, local_attention_window_size: Optional[int] = None,
                 umup_mult: Optional[float] = None):
        super().__init__(head_dim, dropout_p, causal, umup_mult)
        self.masked_softmax_config = masked_softmax_config
        self.num_local_attention_heads = num_local_attention_heads
        self.local_attention_window_size = local_attention_window_size

    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                cumulative_seq_lengths_query: Optional[torch.Tensor],
                cumulative_seq_lengths_key: Optional[torch.Tensor] = None,
                local: Optional[bool] = None,
                doc_ranges: Optional[tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
        """query ``[Tq, h, d]``, key/value ``[Tk, hkv, d]`` (token-major, packed) -> ``[Tq, h, d]``."""
        query, key, value = self._pre(query, key, value)
        use_window = self.local_attention_window_size if (local is None or local) else None
        drop_p = self.dropout_p if self.training else 0.0
        topology = getattr(self, "topology", None)
        out = flash_attention(
            query, key, value, cumulative_seq_lengths_query, cumulative_seq_lengths_key, causal=self.causal,
            scale=self.query_key_scaling_factor, window=use_window, dropout_p=drop_p, doc_ranges=doc_ranges,
            # the kernel draws the mask from the topology's counter-based stream (same on all tensor-parallel ranks,
            # whose heads differ) and recomputes it in the backward pass
            rng_state=topology.kernel_rng if (drop_p > 0.0 and topology is not None and query.is_cuda) else None,
            head_offset=topology.model_parallel_rank * query.shape[1] if topology is not None else 0,
        )
        return self._post(out)


class ParallelSelfAttention(torch.nn.Module):
    def __init__(self, hidden_size: int, num_attention_heads: int, masked_softmax_config: MaskedSoftmaxConfig,
                 causal: bool = True, num_local_attention_heads: int = 0,
                 local_attention_window_size: Optional[int] = None, dropout_attention_probs: float = 0.0,
                 rotary_config: Optional[RotaryConfig] = None,
                 relative_position_embedding_type: RelativePositionEmbeddingType = RelativePositionEmbeddingType.ROTARY,
                 bias: bool = True, device: Optional[torch.device] = None, dtype: torch.dtype = torch.float32,
                 topology: Optional[Topology] = None,
                 init_method: Callable[[torch.Tensor], torch.Tensor] = torch.nn.init.xavier_normal_,
                 bitfit_bias_name: Optional[str] = None, lora_config: Optional[LoRaConfig] = None,
                 norm_type: NormType = NormType.LAYERNORM, key_query_norm: bool = False,
                 layernorm_config: Optional[LayerNormConfig] = None, qkv_in_one: bool = True,
                 num_kv_heads: Optional[int] = None, use_matmul: bool = False, umup_mult: Optional[float] = None,
                 umup_is_first_layer: Optional[bool] = None, umup_is_last_layer: Optional[bool] = None,
                 umup_on_residual: Optional[bool] = None, fp8_config: Optional[Any] = None,
                 fp8_config_dense_out: Optional[Any] = None) -> None:
        super().__init__()
        assert not (topology is not None and device is not None), "cannot specify both device and topology"
        self._device = get_device(topology, device)
        assert hidden_size % num_attention_heads == 0, (
            f"hidden size ({hidden_size}) must be divisible by num_attention_heads ({num_attention_heads})"
        )
        self.hidden_size = hidden_size
        self.hidden_size_per_attention_head = hidden_size // num_attention_heads
        self.num_attention_heads = num_attention_heads
        self.causal = causal
        self.lora_config = lora_config
        self.masked_softmax_config = masked_softmax_config
        self.use_flash_attention = masked_softmax_config.kernel == MaskedSoftmaxKernel.FLASH_ATTENTION
        self.num_local_attention_heads = num_local_attention_heads
        self.local_attention_window_size = local_attention_window_size
        mp = 1 if topology is None else topology.config.model_parallel_size
        if num_local_attention_heads > 0:
            assert self.use_flash_attention, "local attention is currently only supported, with `flash_attention`."
            assert local_attention_window_size is not None, (
                "`local_attention_window_size` needs to be set if `num_local_attention_heads`."
            )
            if num_local_attention_heads != num_attention_heads and mp > 1:
                raise NotImplementedError("Mixed range attention is currently not supported when using tensor parallelism.")
        assert num_attention_heads % mp == 0, (
            f"attention heads ({num_attention_heads}) must be divisible by model parallel size ({mp})"
        )
        self.num_attention_heads_per_partition = num_attention_heads // mp
        self.dtype = dtype
        self.topology = topology
        self.model_parallel_size = mp

        qkv_type = dense_type = None
        if isinstance(umup_is_first_layer, bool):
            qkv_type = UMUP_WEIGHT_TYPE.INPUT_WEIGHT if umup_is_first_layer else UMUP_WEIGHT_TYPE.HIDDEN_WEIGHT
        if isinstance(umup_is_last_layer, bool):
            dense_type = UMUP_WEIGHT_TYPE.OUTPUT_WEIGHT if umup_is_last_layer else UMUP_WEIGHT_TYPE.HIDDEN_WEIGHT

        self.qkv_in_one = qkv_in_one
        self.num_kv_heads = num_kv_heads
        # KV heads fewer than the TP width: every rank keeps full copies of the KV projections
        self.kv_replicated = False
        if num_kv_heads:
            assert not qkv_in_one, "for a differing number of kv heads, qkv cannot be stored in one"
            if num_kv_heads >= mp:
                assert num_kv_heads % mp == 0, f"kv heads ({num_kv_heads}) must be divisible by model parallel size ({mp})"
                self.num_kv_heads_per_partition = num_kv_heads // mp
            else:
                assert mp % num_kv_heads == 0, f"model parallel size ({mp}) must be a multiple of kv heads ({num_kv_heads})"
                self.kv_replicated = True
                self.num_kv_heads_per_partition = num_kv_heads
            self.num_repeat_kv = num_attention_heads // num_kv_heads
        else:
            self.num_kv_heads_per_partition = self.num_attention_heads_per_partition
            self.num_repeat_kv = 1
        kv_features = hidden_size // self.num_repeat_kv

        if lora_config:
            self.lora_merged_state = False
            self.lora_modules = torch.nn.ModuleDict()
            for module_type in lora_config.parallel_modules:
                rep = 1 if module_type in (LoRAModuleType.DENSE, LoRAModuleType.QUERY) else self.num_repeat_kv
                self.lora_modules[f"{module_type.value}_{lora_config.name}"] = ParallelLoRa(
                    in_features=hidden_size, out_features=hidden_size // rep, rank=lora_config.rank,
                    topology=topology, dropout=lora_config.dropout, dtype=dtype, lora_module_type=module_type,
                    alpha=lora_config.alpha, bias=lora_config.bias, kaiming_a=lora_config.kaiming_a,
                    device=None if topology is not None else self._device,
                )

        col = dict(in_features=hidden_size, bias=bias, device=device, dtype=dtype, topology=topology,
                   init_method=init_method, bitfit_bias_name=bitfit_bias_name, parallel_output=True,
                   umup_weight_type=qkv_type, umup_on_residual=umup_on_residual, fp8_config=fp8_config)
        if qkv_in_one:
            self.query_key_value = ColumnParallelLinear(out_features=hidden_size * 3, **col)
        else:
            self.query = ColumnParallelLinear(out_features=hidden_size, **col)
            if self.kv_replicated:
                rep_col = dict(col, topology=None, device=self._device)
                self.key = ColumnParallelLinear(out_features=kv_features, **rep_col)
                self.value = ColumnParallelLinear(out_features=kv_features, **rep_col)
                # replicated parameters: each rank's gradient covers only its own query heads, so the
                # optimizer sums these gradients over the tensor-parallel group before the update
                for lin in (self.key, self.value):
                    for p in lin.parameters():
                        p.core_parameter_meta.is_model_parallel = False  # type: ignore[attr-defined]
                        p.core_parameter_meta.model_parallel_dimension = None  # type: ignore[attr-defined]
                        p.reduce_grad_over_model_parallel = True  # type: ignore[attr-defined]
            else:
                self.key = ColumnParallelLinear(out_features=kv_features, **col)
                self.value = ColumnParallelLinear(out_features=kv_features, **col)

        self.relative_position_embedding_type = relative_position_embedding_type
        self.rotary_embedding: Optional[Union[RotaryEmbedding, RotaryEmbeddingComplex]] = None
        if relative_position_embedding_type == RelativePositionEmbeddingType.ROTARY:
            assert rotary_config is not None
            self.rotary_embedding = RotaryEmbedding(config=rotary_config, device=self._device, dtype=dtype)
        elif relative_position_embedding_type == RelativePositionEmbeddingType.ROTARY_COMPLEX:
            assert rotary_config is not None
            self.rotary_embedding = RotaryEmbeddingComplex(config=rotary_config, device=self._device)
        elif relative_position_embedding_type != RelativePositionEmbeddingType.NONE:
            raise NotImplementedError

        self.key_query_norm = key_query_norm
        self.norm_query: Optional[Union[LayerNorm, RMSNorm]] = None
        self.norm_key: Optional[Union[LayerNorm, RMSNorm]] = None
        if key_query_norm:
            mk = dict(norm_type=norm_type, layernorm_config=layernorm_config,
                      dimensions=self.hidden_size_per_attention_head, device=self._device, dtype=dtype,
                      bitfit_bias_name=bitfit_bias_name)
            self.norm_query = get_norm(**mk)
            self.norm_key = get_norm(**mk)

        self.scaled_dot_product_attention: Union[ScaledDotProductAttention, FlashAttention]
        if self.use_flash_attention:
            self.scaled_dot_product_attention = FlashAttention(
                head_dim=self.hidden_size_per_attention_head, dropout_p=dropout_attention_probs,
                masked_softmax_config=masked_softmax_config, num_local_attention_heads=num_local_attention_heads,
                causal=causal, local_attention_window_size=local_attention_window_size, umup_mult=umup_mult,
            )
            self.scaled_dot_product_attention.topology = topology  # source of the attention-dropout stream
        else:
            self.scaled_dot_product_attention = ScaledDotProductAttention(
                head_dim=self.hidden_size_per_attention_head, dropout_p=dropout_attention_probs,
                masked_softmax_config=masked_softmax_config, causal=causal, umup_mult=umup_mult, use_matmul=use_matmul,
            )

        self.dense = RowParallelLinear(
            in_features=hidden_size, out_features=hidden_size, bias=bias, topology=topology, dtype=dtype,
            device=device, bitfit_bias_name=bitfit_bias_name, init_method=init_method, parallel_input=True,
            parallel_output=(topology.config.sequence_parallel if topology is not None else False),
            umup_weight_type=dense_type, umup_on_residual=umup_on_residual, fp8_config=fp8_config_dense_out,
        )
        self.cache: Dict[int, Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]] = dict()

    # ------------------------------------------------------------------ projections
    def _project_qkv(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """``x [b, s, h]`` -> token-major ``q [T, np, d]``, ``k, v [T, nkv, d]`` (views where possible)."""
        b, s, _ = x.shape
        T = b * s
        d = self.hidden_size_per_attention_head
        npp = self.num_attention_heads_per_partition
        if self.qkv_in_one:
            qkv = self.query_key_value(x).view(T, npp, 3 * d)
            q, k, v = qkv[..., :d], qkv[..., d:2 * d], qkv[..., 2 * d:]
        else:
            q = self.query(x).view(T, npp, d)
            x_kv = x
            if (self.kv_replicated and self.model_parallel_size > 1 and isinstance(x, torch.Tensor)
                    and self.topology is not None and not self.topology.config.sequence_parallel):
                # every rank back-propagates only through the KV heads its own queries read: the input gradient of
                # the replicated projections is a partial sum and is reduced like that of a column-parallel linear
                x_kv = copy_to_tensor_model_parallel_region(x, self.topology)
            k = self.key(x_kv).view(T, -1, d)
            v = self.value(x_kv).view(T, -1, d)
            if self.kv_replicated and k.shape[1] > 1:
                # keep only the KV heads that this rank's query heads read
                r = self.topology.model_parallel_rank if self.topology is not None else 0
                first = (r * npp) // self.num_repeat_kv
                last = ((r + 1) * npp - 1) // self.num_repeat_kv
                k, v = k[:, first:last + 1], v[:, first:last + 1]
        if self.lora_config is not None and not self.lora_merged_state:
            q, k, v = self._apply_lora(x, q, k, v)
        return q, k, v

    def _apply_lora(self, x: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
        assert self.lora_config is not None
        d = self.hidden_size_per_attention_head
        T = x.shape[0] * x.shape[1]
        name = self.lora_config.name
        for key_, module in self.lora_modules.items():
            if key_ == f"dense_{name}":
                continue
            delta = module(x).view(T, -1, d)
            if module.lora_module_type == LoRAModuleType.QUERY:
                q = q + delta
            elif module.lora_module_type == LoRAModuleType.KEY:
                k = k + delta
            elif module.lora_module_type == LoRAModuleType.VALUE:
                v = v + delta
        return q, k, v

    def _qk_norm(self, t: torch.Tensor, norm: torch.nn.Module) -> torch.Tensor:
        # gather heads so that the replicated norm parameters see identical statistics on all ranks
        if self.model_parallel_size > 1 and self.topology is not None:
            full = all_concat(t.transpose(1, 2), self.topology).transpose(1, 2)  # heads -> last dim and back
            return all_shard(norm(full).transpose(1, 2), self.topology).transpose(1, 2)
        return norm(t)

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, cumulative_seq_lengths: Optional[torch.Tensor],
                position_ids: Optional[torch.Tensor],
                cumulative_seq_lengths_key: Optional[torch.Tensor] = None, use_cache: bool = False,
                reset_cache: bool = False, cache_index: int = 0,
                attention_scores_manipulation: Optional[torch.Tensor] = None,
                attentions_score_manipulation_log_additive: Union[bool, List[bool]] = True,
                doc_ranges: Optional[tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
        """``doc_ranges`` (per-token document start / end, int32) may stand in for ``cumulative_seq_lengths`` on
        the fused attention path; it is what a captured CUDA graph passes, since it has a fixed shape."""
        if isinstance(x, SequenceShard) and (use_cache or reset_cache or
                                             (self.lora_config is not None and not self.lora_merged_state)):
            x = x.gathered()  # something besides the projections reads the input
        b, s, _ = x.shape
        T = b * s
        d = self.hidden_size_per_attention_head
        if self._packed_path_ok(x, use_cache, reset_cache):
            hidden = self._packed_attention(x, cumulative_seq_lengths, position_ids, doc_ranges)
            return self._output_projection(hidden)
        q, k, v = self._project_qkv(x)

        if self.key_query_norm:
            assert self.norm_query is not None and self.norm_key is not None
            q = self._qk_norm(q, self.norm_query)
            k = self._qk_norm(k, self.norm_key)

        if self.rotary_embedding is not None:
            if position_ids is not None:
                pos = position_ids.reshape(-1)
            else:
                pos = torch.arange(s, device=x.device, dtype=torch.int32).repeat(b)
            rot = self.rotary_embedding
            q = apply_rotary_tokens(q, pos, rot.dimensions, rot.base, rot.interleaved)
            k = apply_rotary_tokens(k, pos, rot.dimensions, rot.base, rot.interleaved)

        if use_cache:
            if not self.causal:
                raise ValueError("KV caching is only supported for causal attention.")
            assert b == 1, f"KV caching is only supported for batch size 1, got {b}"
            assert cumulative_seq_lengths.numel() == 2 and int(cumulative_seq_lengths[-1]) == T, (
                "sequence packing is not supported with cache"
            )
            if not reset_cache:
                past_k, past_v = self.cache[cache_index]
                assert past_k is not None and past_v is not None
                k = torch.cat((past_k, k), dim=0)
                v = torch.cat((past_v, v), dim=0)
            self.cache[cache_index] = (k, v)
            cumulative_seq_lengths_key = torch.tensor([0, k.shape[0]], device=x.device, dtype=torch.int32)
        elif reset_cache:
            self.cache[cache_index] = (None, None)

        if self.use_flash_attention:
            core = self.scaled_dot_product_attention
            assert isinstance(core, FlashAttention)
            nl = self.num_local_attention_heads
            if nl <= 0 or nl == self.num_attention_heads:
                ctx = core(q, k.contiguous() if use_cache else k, v.contiguous() if use_cache else v,
                           cumulative_seq_lengths, cumulative_seq_lengths_key, local=nl > 0,
                           doc_ranges=None if use_cache else doc_ranges)
            else:  # first `nl` heads attend locally, the rest globally (tensor parallel size 1 only)
                rep = self.num_repeat_kv
                k_full = k.repeat_interleave(rep, dim=1) if rep > 1 else k
                v_full = v.repeat_interleave(rep, dim=1) if rep > 1 else v
                loc = core(q[:, :nl].contiguous(), k_full[:, :nl].contiguous(), v_full[:, :nl].contiguous(),
                           cumulative_seq_lengths, cumulative_seq_lengths_key, local=True)
                glob = core(q[:, nl:].contiguous(), k_full[:, nl:].contiguous(), v_full[:, nl:].contiguous(),
                            cumulative_seq_lengths, cumulative_seq_lengths_key, local=False)
                ctx = torch.cat((loc, glob), dim=1)
        else:
            core2 = self.scaled_dot_product_attention
            assert isinstance(core2, ScaledDotProductAttention)
            rep = q.shape[1] // k.shape[1]
            sk = k.shape[0] // b
            kb = k.view(b, sk, -1, d)
            vb = v.view(b, sk, -1, d)
            if rep > 1:
                kb = kb.repeat_interleave(rep, dim=2)
                vb = vb.repeat_interleave(rep, dim=2)
            ctx = core2(q.view(b, s, -1, d), kb, vb, cumulative_seq_lengths,
                        attention_scores_manipulation=attention_scores_manipulation,
                        attentions_score_manipulation_log_additive=attentions_score_manipulation_log_additive)
        return self._output_projection(ctx.reshape(b, s, -1))

    def _packed_path_ok(self, x: torch.Tensor, use_cache: bool, reset_cache: bool) -> bool:
        """The fused projection -> rotary -> attention path covers training-style self-attention on CUDA with a
        packed qkv weight, all heads global or all local, no adapters, no q/k norm."""
        if not (self.use_flash_attention and self.qkv_in_one and x.is_cuda and x.dtype == torch.bfloat16):
            return False
        if use_cache or reset_cache or self.key_query_norm:
            return False
        if self.lora_config is not None and not self.lora_merged_state:
            return False
        if self.hidden_size_per_attention_head not in (64, 128):
            return False
        if 0 < self.num_local_attention_heads < self.num_attention_heads:
            return False
        core = self.scaled_dot_product_attention
        if core._use_umup or (core.dropout_p > 0.0 and self.training and self.topology is None):
            return False
        from ....ops import _lib

        return _lib.lib_has("sb200_fa_bwd_strided")

    def _packed_attention(self, x: torch.Tensor, cumulative_seq_lengths: Optional[torch.Tensor],
                          position_ids: Optional[torch.Tensor],
                          doc_ranges: Optional[tuple[torch.Tensor, torch.Tensor]]) -> torch.Tensor:
        from ....ops.attention_kernel import dropout_args, packed_qkv_attention

        b, s, _ = x.shape
        d = self.hidden_size_per_attention_head
        qkv = self.query_key_value(x).view(b * s, self.num_attention_heads_per_partition, 3 * d)
        rotary = pos = None
        if self.rotary_embedding is not None:
            rot = self.rotary_embedding
            rotary = (rot.dimensions, rot.base, rot.interleaved)
            pos = (position_ids.reshape(-1) if position_ids is not None
                   else torch.arange(s, device=x.device, dtype=torch.int32).repeat(b))
        core = self.scaled_dot_product_attention
        window = core.local_attention_window_size if self.num_local_attention_heads > 0 else None
        drop_p = core.dropout_p if self.training else 0.0
        drop = dropout_args(drop_p, self.topology.kernel_rng if drop_p > 0.0 else None,
                            self.topology.model_parallel_rank * self.num_attention_heads_per_partition
                            if self.topology is not None else 0)
        ctx = packed_qkv_attention(qkv, pos, rotary, cumulative_seq_lengths, self.causal,
                                   core.query_key_scaling_factor, window, doc_ranges, drop)
        return ctx.reshape(b, s, -1)

    def _output_projection(self, hidden: torch.Tensor) -> torch.Tensor:
        lora_dense = None
        if self.lora_config and not self.lora_merged_state and LoRAModuleType.DENSE in self.lora_config.parallel_modules:
            full = all_concat(hidden, self.topology) if self.model_parallel_size > 1 else hidden
            lora_dense = self.lora_modules[f"dense_{self.lora_config.name}"](full)
        sp = self.topology is not None and self.topology.config.sequence_parallel
        if sp:
            out = self.dense.forward_to_sequence_parallel(hidden)
            if lora_dense is not None:
                # the adapter's output is already summed over the ranks: it joins after the reduction, as this
                # rank's tokens of it (added to the partial sums it would be counted once per rank)
                out = out + shard_to_sequence_parallel_region(lora_dense, self.topology)
            return out
        out = self.dense(hidden)
        if lora_dense is not None:
            out = out + lora_dense
        return out

    # ------------------------------------------------------------------ LoRA merge
    @torch.no_grad()
    def merge_lora_weights(self) -> None:
        assert self.lora_config and self.lora_modules, "Merge of LoRa weights called without proper configuration."
        name = self.lora_config.name
        d = self.hidden_size_per_attention_head
        for key_, module in self.lora_modules.items():
            kind = key_[: -len(name) - 1]
            delta = module.get_delta_weights()
            if kind == "dense":
                self.dense.weight.data += delta.to(self.dense.weight.dtype)
            elif self.qkv_in_one:
                # fused weight rows are interleaved per head as [q_h | k_h | v_h]
                slot = {"query": 0, "key": 1, "value": 2}[kind]
                w = self.query_key_value.weight.data.view(self.num_attention_heads_per_partition, 3, d, -1)
                w[:, slot] += delta.view(self.num_attention_heads_per_partition, d, -1).to(w.dtype)
            else:
                target = getattr(self, kind)
                target.weight.data += delta.to(target.weight.dtype)
        del self.lora_modules
        self.lora_merged_state = True
