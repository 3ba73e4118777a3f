from .rng_tracker import CudaRNGStateTracker
from .topology import Topology
from .topology_config import ActivationCheckpointingType, PipePartitionMethod, TopologyConfig

__all__ = [
    "ActivationCheckpointingType",
    "CudaRNGStateTracker",
    "PipePartitionMethod",
    "Topology",
    "TopologyConfig",
]
