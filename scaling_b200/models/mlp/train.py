"""Entry point of the MLP application: ``python -m scaling_b200.models.mlp.train --payload <b64>`` under
the launcher, or ``main(launch_config)`` from Python (counterpart of examples/mlp_example/train.py)."""

from __future__ import annotations

from typing import Any, Optional

from ...core.logging import logger
from ...core.runner import LaunchConfig
from ...core.trainer import BaseTrainer
from ...parallel.topology import Topology
from .config import MLPConfig
from .data import MNISTDataset, SyntheticClassificationDataset
from .model import MLPContext, init_model, init_optimizer, loss_function, metrics_aggregation_fn


def main(launch_config: LaunchConfig, overwrite_config: Optional[dict] = None,
         return_metrics: bool = False) -> Optional[list[dict[str, Any]]]:
    assert launch_config.payload is not None, "the launcher payload carries the config"
    config_dict = launch_config.overwrite_config_dict_with_launcher_args(dict(launch_config.payload))
    config = MLPConfig.from_dict(config_dict, overwrite_values=overwrite_config)
    topology = Topology(config.topology)
    logger.configure(config.logger, name=f"rank {topology.config.global_rank}", global_rank=topology.config.global_rank)
    context = MLPContext(config=config, topology=topology)
    context.initialize(master_addr=launch_config.master_addr, master_port=str(launch_config.master_port),
                       seed=config.trainer.seed)
    model = init_model(context)
    optimizer = init_optimizer(context, model)
    dataset = None
    if topology.is_io_rank:
        if config.data.synthetic or config.data.mnist_dir is None:
            dataset = SyntheticClassificationDataset(
                n_samples=config.data.n_samples, input_dim=config.architecture.input_dim,
                classes=config.architecture.output_dim, seed=config.trainer.seed,
            )
        else:
            dataset = MNISTDataset(config.data.mnist_dir, train=True, seed=config.trainer.seed)
    trainer = BaseTrainer(
        config=config.trainer, context=context, parallel_module=model, optimizer=optimizer, dataset=dataset,
        sync_batch_to_model_parallel=SyntheticClassificationDataset.sync_batch_to_model_parallel,
        loss_function=loss_function, metrics_aggregation_fn=metrics_aggregation_fn,
    )
    return trainer.run_training(return_metrics=return_metrics)


if __name__ == "__main__":
    main(LaunchConfig.from_launcher_args())
