"""Configuration of the MLP example (step 1 of the walk-through in README.md): ``MLPConfig`` and its sections, defined
in ``scaling_b200.models.mlp.config`` and importable from here as in the example's original layout."""

from scaling_b200.models.mlp.config import MLPArchitectureConfig, MLPConfig, MLPDataConfig, MLPTrainingConfig

__all__ = ["MLPArchitectureConfig", "MLPConfig", "MLPDataConfig", "MLPTrainingConfig"]
