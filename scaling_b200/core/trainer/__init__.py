from .trainer import BaseTrainer
from .trainer_config import TrainerConfig

__all__ = ["BaseTrainer", "TrainerConfig"]
