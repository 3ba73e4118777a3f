from .fp8_config import FP8DType, FP8LinearConfig, FP8MatmulConfig
from .fp8_linear import fp8_linear, saturating_cast

__all__ = ["FP8DType", "FP8LinearConfig", "FP8MatmulConfig", "fp8_linear", "saturating_cast"]
