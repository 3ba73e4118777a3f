"""Single-process pipeline over a list of devices, for inference.

All layers live in one process; consecutive groups of layers sit on consecutive devices and the
activation record is moved at group boundaries.  Tied layer specs become plain specs (weights come
from the checkpoint).  ``forward_with_hidden_state_recorder`` captures outputs of chosen layers or
sub-modules with forward hooks (src/scaling/core/nn/parallel_module/inference_module.py:13-122).
"""

from __future__ import annotations

from dataclasses import dataclass
from functools import partial
from typing import Any, Optional, Sequence, Union

import torch

from ....parallel.topology_config import PipePartitionMethod
from ...data.base_layer_io import BaseLayerIO
from .layer_spec import LayerSpec, TiedLayerSpec
from .partitioned_module import PipePartitionedModule


@dataclass
class RecorderSetting:
    include_modules: Optional[Sequence[str]] = ("",)
    exclude_modules: Optional[Sequence[str]] = None

    def __post_init__(self) -> None:
        assert self.include_modules is None or self.exclude_modules is None, (
            "Cannot specify both include_modules and exclude_modules"
        )

    def wants(self, name: str) -> bool:
        if self.include_modules is not None:
            return name in self.include_modules
        if self.exclude_modules is not None:
            return name not in self.exclude_modules
        return False


class HiddenStateRecorder:
    def __init__(self, module: PipePartitionedModule, recorder_settings_per_layer: dict[int, RecorderSetting]):
        self._module = module
        self.recorder_settings_per_layer = recorder_settings_per_layer
        self.current_record: dict[int, dict[str, Any]] = {k: {} for k in recorder_settings_per_layer}
        self._hooks: list[Any] = []

    def __enter__(self) -> "HiddenStateRecorder":
        self.start_recording()
        return self

    def __exit__(self, *exc: Any) -> None:
        self.stop_recording()

    def record_output(self, module: torch.nn.Module, input: Any, output: Any, layer_index: int, name: str) -> None:
        self.current_record[layer_index][name] = output

    def start_recording(self) -> None:
        for layer_index, setting in self.recorder_settings_per_layer.items():
            for name, sub in self._module._layers[layer_index].named_modules():
                if setting.wants(name):
                    self._hooks.append(sub.register_forward_hook(
                        partial(self.record_output, layer_index=layer_index, name=name)))

    def stop_recording(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []

    def delete_records(self) -> None:
        self.current_record = {k: {} for k in self.recorder_settings_per_layer}


class InferenceModule(PipePartitionedModule):
    def __init__(self, layer_specs: list[LayerSpec], devices: Sequence[Union[int, str, torch.device]] = (0,),
                 pipe_partition_method: PipePartitionMethod = PipePartitionMethod.UNIFORM,
                 pipe_partition_overwrite: Optional[list[int]] = None):
        plain = [
            LayerSpec(s.module_class, *s.args, **s.kwargs) if isinstance(s, TiedLayerSpec) else s for s in layer_specs
        ]
        super().__init__(layer_specs=plain, devices=devices, pipe_partition_method=pipe_partition_method,
                         pipe_partition_overwrite=pipe_partition_overwrite)
        self.eval()

    @torch.no_grad()
    def forward(self, x: BaseLayerIO) -> BaseLayerIO:
        current: Optional[torch.device] = None
        for layer, device in zip(self._layers, self._layer_devices):
            if device != current:
                x.to_(device)
                current = device
            x = layer(x)
        return x

    @torch.no_grad()
    def forward_with_hidden_state_recorder(
        self, x: BaseLayerIO, recorder_settings_per_layer: Optional[dict[int, RecorderSetting]] = None
    ) -> tuple[BaseLayerIO, dict[int, dict[str, Any]]]:
        recorder = HiddenStateRecorder(self, recorder_settings_per_layer or {})
        with recorder:
            x = self.forward(x)
        return x, recorder.current_record
