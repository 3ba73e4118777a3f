from .norms import LayerNorm, LayerNormConfig, LayerNormOptimizationType, NormType, RMSNorm, get_norm

__all__ = ["LayerNorm", "LayerNormConfig", "LayerNormOptimizationType", "NormType", "RMSNorm", "get_norm"]
