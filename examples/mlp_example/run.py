"""Launch the MLP example:  python examples/mlp_example/run.py examples/mlp_example/config.yml

The application itself (config, context, dataset, layers, training script) lives in ``scaling_b200/models/mlp`` and
shows how a model is written against ``scaling_b200.core`` alone: layers derive from ``BaseLayer``, the model is a
list of ``LayerSpec``s handed to ``ParallelModule``, the trainer is ``BaseTrainer``.
"""

import argparse

from scaling_b200.core.logging import logger
from scaling_b200.core.runner import runner_main
from scaling_b200.models.mlp import MLPConfig

if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("config", type=str)
    args = parser.parse_args()
    config = MLPConfig.from_yaml(args.config)
    logger.configure(config=config.logger, name="runner")
    runner_main(config.runner, payload=config.as_dict())
