from .logger_config import LoggerConfig, LogLevel, TensorboardRanksConfig
from .logging import ColorFormatter, DeterminedLogger, Logger, logger

__all__ = ["ColorFormatter", "DeterminedLogger", "Logger", "LoggerConfig", "LogLevel", "TensorboardRanksConfig", "logger"]
