"""Context of the MLP example (step 2 of the walk-through): config + topology + progress counters."""

from scaling_b200.models.mlp.model import MLPContext

__all__ = ["MLPContext"]
