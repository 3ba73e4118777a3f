from .base import TransformerLayerBaseIO, TransformerLayerIO
from .embedding import BaseEmbeddingInput, EmbeddingInput
from .heads import LayerNormWrapper, TransformerEmbeddingHead, TransformerLMHead, TransformerLMHeadTied
from .layer import TransformerLayer

__all__ = ["BaseEmbeddingInput", "EmbeddingInput", "LayerNormWrapper", "TransformerEmbeddingHead",
           "TransformerLMHead", "TransformerLMHeadTied", "TransformerLayer", "TransformerLayerBaseIO",
           "TransformerLayerIO"]
