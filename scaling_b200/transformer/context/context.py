"""Context of the transformer application: the typed config plus the generic run-time state."""

from __future__ import annotations

from ...core.context import BaseContext, DeterminedBaseContext
from ...parallel.topology import Topology
from .config import TransformerConfig


class TransformerContext(DeterminedBaseContext):
    config: TransformerConfig

    def __init__(self, config: TransformerConfig, topology: Topology) -> None:
        super().__init__(config=config, topology=topology)
