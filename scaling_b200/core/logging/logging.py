"""Process-wide logger facade: console, per-rank file, wandb, tensorboard and Determined sinks.

``logger`` is a singleton that works before ``configure`` is called (plain console logging), as
in the reference (src/scaling/core/logging/logging.py:48-246).  Metrics are written only by the
ranks the config selects; all sinks are optional imports.
"""

from __future__ import annotations

import json
import logging as pylog
import sys
from pathlib import Path
from typing import Any, Optional

from ..config import BaseConfig
from .logger_config import LoggerConfig, LogLevel

_LEVELS = {
    LogLevel.DEBUG: pylog.DEBUG,
    LogLevel.INFO: pylog.INFO,
    LogLevel.WARNING: pylog.WARNING,
    LogLevel.ERROR: pylog.ERROR,
    LogLevel.CRITICAL: pylog.CRITICAL,
}
_COLORS = {"DEBUG": "\033[37m", "INFO": "\033[36m", "WARNING": "\033[33m", "ERROR": "\033[31m", "CRITICAL": "\033[41m"}


class ColorFormatter(pylog.Formatter):
    """``[time] [LEVEL] [name] message`` with the level coloured when the stream is a terminal."""

    def __init__(self, name: Optional[str] = None, use_color: bool = True):
        super().__init__()
        self.display_name = name
        self.use_color = use_color

    def format(self, record: pylog.LogRecord) -> str:
        level = record.levelname
        if self.use_color:
            level = f"{_COLORS.get(level, '')}{level}\033[0m"
        who = f" [{self.display_name}]" if self.display_name else ""
        return f"[{self.formatTime(record, '%Y-%m-%d %H:%M:%S')}] [{level}]{who} {record.getMessage()}"


class Logger:
    def __init__(self, config: Optional[LoggerConfig] = None, name: Optional[str] = None,
                 global_rank: Optional[int] = None, tensorboard_ranks: Optional[list[int]] = None):
        self.config = config or LoggerConfig()
        self.global_rank = global_rank
        self._log = pylog.getLogger(f"scaling_b200.{id(self)}")
        self._log.propagate = False
        self._log.handlers.clear()
        self._console = pylog.StreamHandler(sys.stdout)
        self._log.addHandler(self._console)
        self._file: Optional[pylog.Handler] = None
        self._tb = None
        self._wandb = None
        self.set_level(self.config.log_level)
        self.set_formatter(name)
        if self.config.log_dir is not None and global_rank is not None:
            Path(self.config.log_dir).mkdir(parents=True, exist_ok=True)
            self._file = pylog.FileHandler(Path(self.config.log_dir) / f"log_rank_{global_rank}.log")
            self._file.setFormatter(ColorFormatter(name, use_color=False))
            self._log.addHandler(self._file)
        if self.config.use_wandb and self.config.is_rank_in_wandb_ranks(global_rank):
            self._init_wandb()
        self.initialize_tensorboard_writer(self.config, tensorboard_ranks)

    # ---- sinks
    def _init_wandb(self) -> None:
        try:
            import wandb
        except ImportError:  # pragma: no cover
            self.warning("wandb requested but not installed; metrics go to the console only")
            return
        wandb.login(key=self.config.wandb_api_key, host=self.config.wandb_host)
        self._wandb = wandb.init(
            project=self.config.wandb_project,
            entity=self.config.wandb_team,
            group=self.config.wandb_group,
            name=f"rank-{self.global_rank}",
            dir=str(self.config.log_dir) if self.config.log_dir else None,
        )

    def initialize_tensorboard_writer(self, config: LoggerConfig, tensorboard_ranks: Optional[list[int]]) -> None:
        if not config.use_tensorboard or self.global_rank is None:
            return
        ranks = tensorboard_ranks if tensorboard_ranks is not None else [0]
        if self.global_rank not in ranks:
            return
        try:
            from torch.utils.tensorboard import SummaryWriter
        except Exception:  # pragma: no cover
            self.warning("tensorboard requested but not importable")
            return
        self._tb = SummaryWriter(log_dir=str(Path(config.log_dir) / f"tensorboard_rank_{self.global_rank}"))

    def set_level(self, log_level: LogLevel) -> None:
        self._log.setLevel(_LEVELS[log_level])

    def set_formatter(self, name: Optional[str] = None) -> None:
        self._console.setFormatter(ColorFormatter(name, use_color=sys.stdout.isatty()))

    # ---- metrics / config
    def log_metrics(self, metrics: dict[str, Any], step: int, to_info: bool = True, to_wandb: bool = True) -> None:
        if not self.config.is_rank_in_metrics_ranks(self.global_rank) and self.global_rank is not None:
            return
        plain = {k: (v.item() if hasattr(v, "item") else v) for k, v in metrics.items()}
        if to_info:
            self.info(json.dumps({"step": step, **plain}, default=str))
        if self._wandb is not None and to_wandb:
            self._wandb.log(plain, step=step)
        if self._tb is not None:
            for k, v in plain.items():
                if isinstance(v, (int, float)):
                    self._tb.add_scalar(k, v, step)

    def log_config(self, config: BaseConfig) -> None:
        self.log_config_dict(config.as_dict())

    def log_config_dict(self, config_dict: dict) -> None:
        self.info("config: " + json.dumps(config_dict, default=str))
        if self._wandb is not None:
            self._wandb.config.update(config_dict, allow_val_change=True)
        if self._tb is not None:
            self._tb.add_text("config", json.dumps(config_dict, default=str, indent=2))

    # ---- plain logging
    def debug(self, msg: object) -> None:
        self._log.debug(msg)

    def info(self, msg: object) -> None:
        self._log.info(msg)

    def warning(self, msg: object) -> None:
        self._log.warning(msg)

    def error(self, msg: object) -> None:
        self._log.error(msg)

    def critical(self, msg: object) -> None:
        self._log.critical(msg)


class DeterminedLogger(Logger):
    """Logger that additionally reports metrics through a Determined core context."""

    def __init__(self, config: LoggerConfig, determined_context: Any, determined_profiler: Any = None,
                 name: Optional[str] = None, global_rank: Optional[int] = None,
                 tensorboard_ranks: Optional[list[int]] = None):
        self.determined_context = determined_context
        self.determined_profiler = determined_profiler
        super().__init__(config, name=name, global_rank=global_rank, tensorboard_ranks=tensorboard_ranks)

    def log_metrics(self, metrics: dict[str, Any], step: int, to_info: bool = True, to_wandb: bool = True) -> None:
        super().log_metrics(metrics, step, to_info=to_info, to_wandb=to_wandb)
        if self.determined_context is not None and self.config.is_rank_in_determined_metrics_ranks(self.global_rank):
            train = {k: v for k, v in metrics.items() if not k.startswith("evaluation")}
            evaluation = {k: v for k, v in metrics.items() if k.startswith("evaluation")}
            if train:
                self.determined_context.train.report_training_metrics(steps_completed=step, metrics=train)
            if evaluation:
                self.determined_context.train.report_validation_metrics(steps_completed=step, metrics=evaluation)


class _LoggerSingleton:
    """Forwards every attribute to the currently configured Logger."""

    def __init__(self) -> None:
        self._impl: Logger = Logger()

    def configure(self, config: LoggerConfig, name: Optional[str] = None, global_rank: Optional[int] = None,
                  tensorboard_ranks: Optional[list[int]] = None) -> None:
        self._impl = Logger(config, name=name, global_rank=global_rank, tensorboard_ranks=tensorboard_ranks)

    def configure_determined(self, config: LoggerConfig, name: Optional[str] = None, global_rank: Optional[int] = None,
                             determined_context: Any = None, tensorboard_ranks: Optional[list[int]] = None,
                             determined_profiler: Any = None) -> None:
        """Argument order of src/scaling/core/logging/logging.py:224-233; without a context the Determined sink
        stays silent."""
        self._impl = DeterminedLogger(config, determined_context, determined_profiler, name=name,
                                      global_rank=global_rank, tensorboard_ranks=tensorboard_ranks)

    def __getattr__(self, name: str) -> Any:
        return getattr(self._impl, name)


logger = _LoggerSingleton()
