from .attention import (
    FlashAttention,
    ParallelSelfAttention,
    RelativePositionEmbeddingType,
    ScaledDotProductAttention,
    cumulative_seq_lengths_to_dense_attention_mask,
    get_max_seq_length,
)

__all__ = ["FlashAttention", "ParallelSelfAttention", "RelativePositionEmbeddingType", "ScaledDotProductAttention",
           "cumulative_seq_lengths_to_dense_attention_mask", "get_max_seq_length"]
