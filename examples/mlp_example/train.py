"""Training entry point of the MLP example (step 6 of the walk-through); the launcher starts this module on every
rank: ``python -m examples.mlp_example.train``."""

from scaling_b200.core.runner import LaunchConfig
from scaling_b200.models.mlp.train import main

__all__ = ["main"]

if __name__ == "__main__":
    main(LaunchConfig.from_launcher_args())
