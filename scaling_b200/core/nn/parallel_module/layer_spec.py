"""Deferred layer constructors.

A model is described as a list of ``LayerSpec(module_class, *args, **kwargs)``; each pipeline stage
instantiates only the layers it owns, directly on its device.  ``TiedLayerSpec`` marks layers that
share parameters (``tied_weight_attributes``) with every other spec of the same ``key``
(reference: src/scaling/core/nn/parallel_module/layer_spec.py:8-32).
"""

from __future__ import annotations

from typing import Any, Optional

import torch


class LayerSpec:
    def __init__(self, module_class: type, *args: Any, **kwargs: Any) -> None:
        if not isinstance(module_class, type) or not issubclass(module_class, torch.nn.Module):
            raise TypeError(f"LayerSpec needs a torch.nn.Module subclass, got {module_class!r}")
        self.module_class = module_class
        self.args = args
        self.kwargs = kwargs

    def initialize(self, device: Optional[torch.device] = None) -> torch.nn.Module:
        module = self.module_class(*self.args, **self.kwargs)
        return module if device is None else module.to(device)

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.module_class.__name__})"


class TiedLayerSpec(LayerSpec):
    """``TiedLayerSpec(module_class, key, tied_weight_attributes, *args, **kwargs)``; the three may also be given by
    keyword or in the order ``(key, tied_weight_attributes, module_class)`` of
    src/scaling/core/nn/parallel_module/layer_spec.py:19-32."""

    def __init__(self, *args: Any, **kwargs: Any):
        names = ("module_class", "key", "tied_weight_attributes")
        given = {n: kwargs.pop(n) for n in names if n in kwargs}
        rest = list(args)
        order = names if (rest and isinstance(rest[0], type)) else ("key", "tied_weight_attributes", "module_class")
        for n in order:
            if n not in given:
                if not rest:
                    raise TypeError(f"TiedLayerSpec: missing argument '{n}'")
                given[n] = rest.pop(0)
        super().__init__(given["module_class"], *rest, **kwargs)
        self.key = given["key"]
        attributes = list(given["tied_weight_attributes"])
        assert len(set(attributes)) == len(attributes), f"duplicates in tied_weight_attributes: {attributes}"
        self.tied_weight_attributes = attributes
