from .config import TransformerArchitectureConfig, TransformerConfig
from .context import TransformerContext

__all__ = ["TransformerArchitectureConfig", "TransformerConfig", "TransformerContext"]
