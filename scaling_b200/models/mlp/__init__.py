from .config import MLPArchitectureConfig, MLPConfig
from .data import MLPDatasetBatch, MNISTDataset, SyntheticClassificationDataset
from .model import MLPContext, get_layer_specs, init_model, init_optimizer, loss_function, metrics_aggregation_fn

__all__ = ["MLPArchitectureConfig", "MLPConfig", "MLPContext", "MLPDatasetBatch", "MNISTDataset",
           "SyntheticClassificationDataset", "get_layer_specs", "init_model", "init_optimizer", "loss_function",
           "metrics_aggregation_fn"]
