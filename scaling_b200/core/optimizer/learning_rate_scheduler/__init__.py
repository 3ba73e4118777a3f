from .learning_rate_scheduler import LearningRateDecayStyle, LearningRateScheduler, LearningRateSchedulerConfig

__all__ = ["LearningRateDecayStyle", "LearningRateScheduler", "LearningRateSchedulerConfig"]
