"""Logger configuration (same fields as src/scaling/core/logging/logger_config.py:28-143)."""

from __future__ import annotations

import os
import re
import warnings
from datetime import datetime
from enum import Enum
from pathlib import Path
from typing import Any, Optional

from pydantic import Field, model_validator

from ..config import BaseConfig

_STAMP = "%Y-%m-%d-%H-%M-%S"
_STAMP_RE = re.compile(r"^\d{4}-\d{2}-\d{2}-\d{2}-\d{2}-\d{2}$")


class LogLevel(Enum):
    DEBUG = "debug"
    INFO = "info"
    WARNING = "warning"
    ERROR = "error"
    CRITICAL = "critical"


class TensorboardRanksConfig(BaseConfig):
    pipe_parallel_rank: Optional[int] = Field(None, description="select ranks with this pipe coordinate")
    data_parallel_rank: Optional[int] = Field(None, description="select ranks with this data coordinate")
    model_parallel_rank: Optional[int] = Field(None, description="select ranks with this model coordinate")


def looks_like_timestamp(name: str) -> bool:
    if _STAMP_RE.match(name):
        return True
    try:
        from dateutil.parser import parse  # optional dependency

        parse(name, fuzzy=False)
        return True
    except Exception:
        return False


def rank_selected(rank: Optional[int], ranks: Optional[list[int]]) -> bool:
    if rank is None:
        return False
    return rank in ranks if ranks is not None else rank == 0


def check_if_in_rank(target_rank: Optional[int], ranks: Optional[list[int]]) -> bool:
    """Name and signature of src/scaling/core/logging/logger_config.py:118."""
    return rank_selected(target_rank, ranks)


class LoggerConfig(BaseConfig):
    log_level: LogLevel = Field(LogLevel.INFO, description="console / file log level")
    log_dir: Optional[Path] = Field(None, description="directory for per-rank log files and tensorboard events")
    metrics_ranks: Optional[list[int]] = Field(None, description="global ranks that write metrics (default: rank 0)")
    use_wandb: bool = Field(False, description="report metrics to Weights & Biases")
    wandb_ranks: Optional[list[int]] = Field(None, description="global ranks that write to wandb (default: rank 0)")
    wandb_host: str = Field("https://api.wandb.ai", description="url of the wandb host")
    wandb_team: str = Field("aleph-alpha", description="wandb entity")
    wandb_project: str = Field("aleph-alpha-scaling", description="wandb project name")
    wandb_group: str = Field("debug", description="wandb group name")
    wandb_api_key: Optional[str] = Field(None, description="wandb api key; falls back to WANDB_API_KEY")
    use_tensorboard: bool = Field(False, description="write tensorboard event files into log_dir")
    tensorboard_ranks: Optional[list[int] | TensorboardRanksConfig] = Field(
        None, description="ranks that write tensorboard events: a list, a coordinate selector, or rank 0"
    )
    determined_metrics_ranks: Optional[list[int]] = Field(None, description="ranks reporting to Determined")

    @model_validator(mode="before")
    @classmethod
    def _normalise(cls, values: Any) -> Any:
        if not isinstance(values, dict):
            return values
        values = dict(values)
        if values.get("use_tensorboard", False) and values.get("log_dir") is None:
            warnings.warn("Setting 'use_tensorboard' to False because no 'log_dir' is defined.")
            values["use_tensorboard"] = False
        log_dir = values.get("log_dir")
        if log_dir is not None:
            log_dir = Path(log_dir)
            if not looks_like_timestamp(log_dir.name):
                log_dir = log_dir / datetime.now().strftime(_STAMP)
            values["log_dir"] = log_dir
        group = values.get("wandb_group")
        if group is not None and not looks_like_timestamp("-".join(group.split("-")[-6:])):
            values["wandb_group"] = group + "-" + datetime.now().strftime(_STAMP)
        key = values.get("wandb_api_key") or os.getenv("WANDB_API_KEY")
        if values.get("use_wandb", False) and not key:
            raise ValueError("If 'use_wandb' is set to True a wandb api key needs to be provided.")
        values["wandb_api_key"] = key
        return values

    def is_rank_in_wandb_ranks(self, rank: Optional[int]) -> bool:
        return rank_selected(rank, self.wandb_ranks)

    def is_rank_in_metrics_ranks(self, rank: Optional[int]) -> bool:
        return rank_selected(rank, self.metrics_ranks)

    def is_rank_in_determined_metrics_ranks(self, rank: Optional[int]) -> bool:
        return rank_selected(rank, self.determined_metrics_ranks)
