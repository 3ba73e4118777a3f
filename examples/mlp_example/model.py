"""Layers, layer specs, loss and optimizer of the MLP example (steps 4 and 5 of the walk-through)."""

from scaling_b200.models.mlp.model import (
    MLPBaseLayer,
    MLPLayerIO,
    MLPLinearColumnParallel,
    MLPLinearRowParallel,
    get_layer_specs,
    init_model,
    init_optimizer,
    loss_function,
    metrics_aggregation_fn,
)

__all__ = ["MLPBaseLayer", "MLPLayerIO", "MLPLinearColumnParallel", "MLPLinearRowParallel", "get_layer_specs",
           "init_model", "init_optimizer", "loss_function", "metrics_aggregation_fn"]
