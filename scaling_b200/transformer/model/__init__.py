from .layers import TransformerLayerIO
from .model import (
    TransformerParallelModule,
    get_parameter_groups,
    get_transformer_layer_specs,
    init_model,
    init_optimizer,
    metrics_aggregation_fn,
)

__all__ = ["TransformerLayerIO", "TransformerParallelModule", "get_parameter_groups", "get_transformer_layer_specs",
           "init_model", "init_optimizer", "metrics_aggregation_fn"]
