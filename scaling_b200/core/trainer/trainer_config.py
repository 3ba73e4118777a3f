"""Trainer settings (fields of src/scaling/core/trainer/trainer_config.py:10-88)."""

from __future__ import annotations

from pathlib import Path
from typing import Any, List, Optional

from pydantic import Field

from ..config import BaseConfig
from ..logging.tensor_statistics_recorder import TensorStatisticsRecorderConfig


class TrainerConfig(BaseConfig):
    save_dir: Optional[Path] = Field(None, description="directory for saving checkpoints")
    save_interval: Optional[int] = Field(None, description="save a checkpoint every n steps (needs save_dir)")
    load_dir: Optional[Path] = Field(None, description="directory for loading checkpoints")
    train_iterations: Optional[int] = Field(None, description="train for this number of iterations")
    assert_checkpoint_loaded: bool = Field(True, description="fail if load_dir is set but nothing could be loaded")
    load_optimizer_states: bool = Field(True, description="load optimizer states on checkpoint load")
    delete_past_optimizer_states: bool = Field(
        True, description="after saving checkpoint n, delete the optimizer states of checkpoints < n"
    )
    load_context: bool = Field(True, description="load iterations / consumed samples / RNG states on checkpoint load")
    allowed_missing_keys_in_checkpoint: Optional[List[str]] = Field(
        None, description="regexes of parameters that may be absent from a checkpoint (e.g. new adapters)"
    )
    allowed_unexpected_keys_in_checkpoint: Optional[List[str]] = Field(
        None, description="regexes of checkpoint entries that may be ignored"
    )
    ignore_keys_in_checkpoint: Optional[List[str]] = Field(
        None, description="regexes of parameters whose checkpoint values are not loaded (re-initialise them)"
    )
    merge_lora_after_loading_checkpoint: Optional[bool] = Field(
        False, description="fold LoRA adapters into the base weights after loading"
    )
    seed: int = Field(42, description="seed of the data order")
    dataloader_num_workers: int = Field(0, description="worker processes of the data loader")
    dataloader_pin_memory: bool = Field(True, description="collate into pinned host memory")
    dataloader_prefetch_factor: Optional[int] = Field(None, description="batches prefetched per worker")
    eval_iterations: int = Field(1, description="evaluation steps per evaluation")
    eval_interval: Optional[int] = Field(None, description="evaluate every n steps")
    separate_file_for_parameters: Optional[List[str]] = Field(
        None, description="parameters whose name contains one of these strings go to separate checkpoint files"
    )
    tensor_statistics_recorder_config: Optional[TensorStatisticsRecorderConfig] = Field(
        None, description="configuration for recording tensor statistics"
    )
