"""Import alias: code written against ``scaling.core`` / ``scaling.transformer`` runs on ``scaling_b200``.

Opt in by putting this directory's parent on the path::

    PYTHONPATH=compat python examples/mlp_example/run.py ...

``import scaling.core``, ``from scaling.core.topology import Topology``, ``from scaling.transformer.context import
TransformerConfig`` and so on then resolve to the modules of ``scaling_b200`` (the same module objects: classes
compare identical under both names).  Modules that ``scaling_b200`` keeps in differently named files are mapped in
``RENAMED`` below.  The package deliberately does not sit at the repository root: an installed copy of the original
``scaling`` package elsewhere on the path must stay importable under its own name when this directory is not listed.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys
from typing import Optional

TARGET = "scaling_b200"

# module paths of the original package whose content lives in another module here
RENAMED = {
    "scaling.core.topology": "scaling_b200.parallel",
    "scaling.core.topology.topology": "scaling_b200.parallel.topology",
    "scaling.core.topology.topology_config": "scaling_b200.parallel.topology_config",
    "scaling.core.topology.rng_tracker": "scaling_b200.parallel.rng_tracker",
    "scaling.core.nn.linear.column_parallel_linear": "scaling_b200.core.nn.linear.parallel_linear",
    "scaling.core.nn.linear.row_parallel_linear": "scaling_b200.core.nn.linear.parallel_linear",
    "scaling.core.nn.lora_config": "scaling_b200.core.nn.lora",
    "scaling.core.nn.rotary_config": "scaling_b200.core.nn.rotary",
    "scaling.core.nn.masked_softmax.masked_softmax_config": "scaling_b200.core.nn.masked_softmax.masked_softmax",
    "scaling.core.nn.norm.get_norm": "scaling_b200.core.nn.norm.norms",
    "scaling.core.nn.norm.layernorm": "scaling_b200.core.nn.norm.norms",
    "scaling.core.nn.norm.layernorm_config": "scaling_b200.core.nn.norm.norms",
    "scaling.core.nn.norm.rms_norm": "scaling_b200.core.nn.norm.norms",
    "scaling.core.nn.pipeline_schedule.base": "scaling_b200.core.nn.pipeline_schedule.instructions",
    "scaling.core.nn.pipeline_schedule.train": "scaling_b200.core.nn.pipeline_schedule.schedules",
    "scaling.core.nn.pipeline_schedule.inference": "scaling_b200.core.nn.pipeline_schedule.schedules",
    "scaling.core.optimizer.learning_rate_scheduler.learning_rate_scheduler_config":
        "scaling_b200.core.optimizer.learning_rate_scheduler.learning_rate_scheduler",
    "scaling.core.optimizer.loss_scaler_config": "scaling_b200.core.optimizer.loss_scaler",
    "scaling.core.optimizer.parameter_group_config": "scaling_b200.core.optimizer.optimizer_config",
    "scaling.core.logging.color_formatter": "scaling_b200.core.logging.logging",
    "scaling.core.utils.determined_utils": "scaling_b200.core.determined.core",
    "scaling.transformer.data.text_dataset_item": "scaling_b200.transformer.data.dataset_item",
    "scaling.transformer.model.layers.embedding_head": "scaling_b200.transformer.model.layers.heads",
    "scaling.transformer.model.layers.layernorm": "scaling_b200.transformer.model.layers.heads",
    "scaling.transformer.model.layers.lm_head": "scaling_b200.transformer.model.layers.heads",
    "scaling.transformer.model.layers.lm_head_tied": "scaling_b200.transformer.model.layers.heads",
}


def _real_name(alias: str) -> str:
    if alias in RENAMED:
        return RENAMED[alias]
    return TARGET + alias[len("scaling"):]


class _AliasLoader(importlib.abc.Loader):
    """Hands out the already imported module of ``scaling_b200`` under its alias name."""

    def __init__(self, real: str):
        self.real = real
        self._spec = None

    def create_module(self, spec):  # type: ignore[no-untyped-def]
        module = importlib.import_module(self.real)
        self._spec = module.__spec__  # the import machinery re-labels the module; put its own spec back afterwards
        return module

    def exec_module(self, module) -> None:  # type: ignore[no-untyped-def]
        if self._spec is not None:
            module.__spec__ = self._spec


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname: str, path=None, target=None):  # type: ignore[no-untyped-def]
        if not fullname.startswith("scaling."):
            return None
        real = _real_name(fullname)
        try:
            found = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            found = None
        if found is None:
            return None
        return importlib.util.spec_from_loader(fullname, _AliasLoader(real),
                                               is_package=found.submodule_search_locations is not None)


def _install() -> None:
    if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
        sys.meta_path.insert(0, _AliasFinder())


_install()


def __getattr__(name: str) -> Optional[object]:
    # `scaling.core`, `scaling.transformer` as attributes of the package
    try:
        return importlib.import_module(f"scaling.{name}")
    except ImportError as e:
        raise AttributeError(name) from e
