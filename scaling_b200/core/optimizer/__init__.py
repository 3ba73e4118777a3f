from .base import BaseOptimizer, OptimizerStepOutput
from .learning_rate_scheduler import LearningRateDecayStyle, LearningRateScheduler, LearningRateSchedulerConfig
from .loss_scaler import LossScaler, LossScalerConfig
from .optimizer import Optimizer
from .optimizer_config import OptimizerConfig, OptimizerParamGroupConfig
from .parameter_group import OptimizerParamGroup

__all__ = ["BaseOptimizer", "LearningRateDecayStyle", "LearningRateScheduler", "LearningRateSchedulerConfig",
           "LossScaler", "LossScalerConfig", "Optimizer", "OptimizerConfig", "OptimizerParamGroup",
           "OptimizerParamGroupConfig", "OptimizerStepOutput"]
