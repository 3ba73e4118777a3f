"""Settings for blending several datasets (fields of src/scaling/core/data/blended_dataset_config.py:16-106)."""

from __future__ import annotations

from pathlib import Path
from typing import List, Optional

from pydantic import Field

from ..config import BaseConfig


class BlendedDatasetConfig(BaseConfig):
    weight_by_num_documents: bool = Field(
        True, description="derive weights from document counts (p^alpha re-normalised); overrides explicit weights"
    )
    weighted_sampler_alpha: float = Field(
        1.0, description="alpha of weight_by_num_documents: 1 = proportional to size, 0 = equal, large = favour big sets"
    )
    weights: Optional[List[float]] = Field(None, description="explicit weights, one per dataset, in dataset order")
    weight_examples_proportional: bool = Field(
        False, description="examples-proportional mixing with rate limit K and temperature T (T5 paper, page 31)"
    )
    ep_maximum: Optional[int] = Field(None, description="rate limit K of examples-proportional mixing")
    ep_temperature: float = Field(1.0, description="temperature T of examples-proportional mixing")
    minimum_dataset_size: int = Field(0, description="minimal size of the blended dataset")
    cache_directory: Optional[Path] = Field(None, description="directory of the blended index (needed for > 1 dataset)")
    shuffle_dataset_indices: bool = Field(False, description="shuffle the blended index after creation")
    load_dataset_indices_to_memory: bool = Field(False, description="read the index into memory instead of mmap")
