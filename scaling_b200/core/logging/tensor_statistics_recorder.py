"""Periodic statistics of activations, gradients and parameters (src/scaling/core/logging/tensor_statistics_recorder.py:24-486).

While ``TensorStatisticsRecorder.trace()`` is active, every module's forward output and full-backward gradient, every
parameter (value now, gradient when it arrives) and every tensor passed to ``tensor_tracker.trace_tensor`` is reduced
to the configured statistics and logged under ``activation_statistics/…``, ``parameter_statistics/…`` and
``tensor_statistics/…``.  Which statistics apply to which name is decided by the first matching glob pattern.
A traced step runs eagerly (the captured training step has no Python hooks).
"""

from __future__ import annotations

import enum
import fnmatch
from collections import defaultdict
from contextlib import contextmanager
from functools import partial
from typing import Any, Callable, Iterator, Literal, Optional

import torch
from pydantic import Field

from ..config import BaseConfig

E4M3_SMALLEST = 2.0 ** -9    # smallest positive subnormal of float8 e4m3
E5M2_SMALLEST = 2.0 ** -16   # smallest positive subnormal of float8 e5m2


class TensorStatistics(enum.Enum):
    L1 = "l1"
    MEAN = "mean"
    STD = "std"
    SKEW = "skew"
    KURTOSIS = "kurtosis"
    MAX = "max"
    MIN = "min"
    MEDIAN = "median"
    ABS_STD = "abs_std"
    ABS_MAX = "abs_max"
    ABS_MIN = "abs_min"
    ABS_MEDIAN = "abs_median"
    ENTROPY = "entropy"                      # of probability rows (attention entropy collapse, arXiv 2309.14322 §3.1.1)
    PCT_ZERO = "pct_zero"
    PCT_UNDERFLOW_E4M3 = "pct_underflow_e4m3"
    PCT_UNDERFLOW_E5M2 = "pct_underflow_e5m2"
    PCT_POSINF = "pct_posinf"
    PCT_NEGINF = "pct_neginf"
    PCT_NAN = "pct_nan"
    MAX_SPARSITY = "max_sparsity"            # outlier measures of the OLMo stability study
    NORM_SPARSITY = "norm_sparsity"
    QUANTILE_1 = "quantile_1"
    QUANTILE_10 = "quantile_10"
    QUANTILE_25 = "quantile_25"
    QUANTILE_75 = "quantile_75"
    QUANTILE_90 = "quantile_90"
    QUANTILE_99 = "quantile_99"
    ABS_QUANTILE_1 = "abs_quantile_1"
    ABS_QUANTILE_10 = "abs_quantile_10"
    ABS_QUANTILE_25 = "abs_quantile_25"
    ABS_QUANTILE_75 = "abs_quantile_75"
    ABS_QUANTILE_90 = "abs_quantile_90"
    ABS_QUANTILE_99 = "abs_quantile_99"


DEFAULT_STATISTICS = [TensorStatistics.MEAN, TensorStatistics.STD, TensorStatistics.L1, TensorStatistics.ABS_STD,
                      TensorStatistics.MAX, TensorStatistics.MIN, TensorStatistics.MEDIAN, TensorStatistics.ABS_MAX,
                      TensorStatistics.ABS_MIN, TensorStatistics.ABS_MEDIAN]


def _quantile(x: torch.Tensor, q: float) -> float:
    flat = x.float().flatten()
    if flat.numel() > 2 ** 24:  # torch.quantile's input limit: an evenly strided subsample keeps the estimate
        flat = flat[:: flat.numel() // 2 ** 24 + 1]
    return flat.quantile(q).item()


def _standardised_moment(x: torch.Tensor, power: float, correction: int) -> torch.Tensor:
    xf = x.float()
    return torch.mean(torch.pow((xf - xf.mean()) / xf.std(correction=correction), power))


def _max_sparsity(x: torch.Tensor) -> float:
    a = x.abs().float()
    med = a.median()
    return ((a.max() - med) / med).item()


TENSOR_STATISTICS_FUNCTIONS: dict[TensorStatistics, Callable[[torch.Tensor], float]] = {
    TensorStatistics.MEAN: lambda x: x.mean().item(),
    TensorStatistics.STD: lambda x: x.std().item(),
    TensorStatistics.SKEW: lambda x: _standardised_moment(x, 3.0, 1).item(),
    TensorStatistics.KURTOSIS: lambda x: (_standardised_moment(x, 4.0, 0) - 3.0).item(),
    TensorStatistics.L1: lambda x: (x.norm(p=1) / x.numel()).item(),
    TensorStatistics.ABS_STD: lambda x: x.abs().std().item(),
    TensorStatistics.MAX: lambda x: x.max().item(),
    TensorStatistics.MIN: lambda x: x.min().item(),
    TensorStatistics.MEDIAN: lambda x: x.float().median().item(),
    TensorStatistics.ABS_MAX: lambda x: x.abs().max().item(),
    TensorStatistics.ABS_MIN: lambda x: x.abs().min().item(),
    TensorStatistics.ABS_MEDIAN: lambda x: x.abs().float().median().item(),
    TensorStatistics.ENTROPY: lambda x: -torch.sum(x * torch.log(x + 1e-9), dim=-1).mean().item(),
    TensorStatistics.PCT_ZERO: lambda x: 1.0 - (x.count_nonzero() / x.numel()).item(),
    TensorStatistics.PCT_UNDERFLOW_E4M3: lambda x: (torch.count_nonzero(x.abs() <= E4M3_SMALLEST) / x.numel()).item(),
    TensorStatistics.PCT_UNDERFLOW_E5M2: lambda x: (torch.count_nonzero(x.abs() <= E5M2_SMALLEST) / x.numel()).item(),
    TensorStatistics.PCT_POSINF: lambda x: (x.isposinf().sum() / x.numel()).item(),
    TensorStatistics.PCT_NEGINF: lambda x: (x.isneginf().sum() / x.numel()).item(),
    TensorStatistics.PCT_NAN: lambda x: (x.isnan().sum() / x.numel()).item(),
    TensorStatistics.MAX_SPARSITY: _max_sparsity,
    TensorStatistics.NORM_SPARSITY: lambda x: (x.numel() ** 0.5 * x.float().norm(p=2) / x.float().norm(p=1)).item(),
}
for _q in (1, 10, 25, 75, 90, 99):
    TENSOR_STATISTICS_FUNCTIONS[TensorStatistics(f"quantile_{_q}")] = partial(lambda x, q: _quantile(x, q), q=_q / 100)
    TENSOR_STATISTICS_FUNCTIONS[TensorStatistics(f"abs_quantile_{_q}")] = partial(lambda x, q: _quantile(x.abs(), q), q=_q / 100)


def statistics_fcts_for_name_pattern(statistics_config: list[tuple[str, list[TensorStatistics]]],
                                     name_pattern: str) -> Optional[dict[str, Callable]]:
    """Statistic functions of the first pattern that matches ``name_pattern``; None if no pattern does."""
    for pattern, stats in statistics_config:
        if fnmatch.fnmatch(name_pattern, pattern):
            return {s.value: TENSOR_STATISTICS_FUNCTIONS[s] for s in stats}
    return None


class TensorStatisticsRecorderConfig(BaseConfig):
    interval: int = Field(100, description="trace metrics every interval steps")
    statistics: list[tuple[str, list[TensorStatistics]]] = Field(
        default_factory=lambda: [("*", list(DEFAULT_STATISTICS))],
        description="glob patterns on metric names -> statistics to record for matching names; first match wins",
    )
    include_module_type: bool = Field(False, description="put the module class into activation metric names")


class _TensorTracker:
    """Process-wide registry through which model code can expose intermediate tensors:
    ``tensor_tracker.trace_tensor(t, "name")`` is a no-op unless a recorder is tracing."""

    _instance: Optional["_TensorTracker"] = None

    def __new__(cls) -> "_TensorTracker":
        if cls._instance is None:
            inst = super().__new__(cls)
            inst.hooks = []
            inst.backward_hooks = []
            inst.name_counter = defaultdict(int)
            cls._instance = inst
        return cls._instance

    def trace_tensor(self, tensor: torch.Tensor, name: str) -> None:
        for hook in self.hooks:
            full = f"tensor_statistics/counter.{self.name_counter[name]}.{name}"
            hook(tensor=tensor, name=full, mode="forward")
            if tensor.requires_grad:
                self.backward_hooks.append(tensor.register_hook(partial(self._backward, hook, full)))
        self.name_counter[name] += 1

    @staticmethod
    def _backward(hook: Callable, name: str, grad: torch.Tensor) -> None:
        hook(tensor=grad, name=name, mode="backward")

    @contextmanager
    def register_hook(self, hook_fn: Callable) -> Iterator[None]:
        try:
            self.hooks.append(hook_fn)
            yield
        finally:
            self.hooks = []
            for h in self.backward_hooks:
                h.remove()
            self.backward_hooks = []
            self.name_counter = defaultdict(int)


tensor_tracker = _TensorTracker()


class TensorStatisticsRecorder:
    def __init__(self, config: TensorStatisticsRecorderConfig, context: Any, model: Any, logger: Any = None):
        from . import logger as default_logger

        self.config = TensorStatisticsRecorderConfig.from_dict(config) if isinstance(config, dict) else config
        self.context = context
        self.model = model
        self.logger = logger if logger is not None else default_logger
        self.module_to_name_dict = {mod: name for name, mod in model.named_modules()}

    # ------------------------------------------------------------------ hooks
    def register_parameter_hooks(self) -> list:
        """Record every parameter now ("forward") and hook its gradient ("backward"); returns the hook handles."""
        hooks = []
        if hasattr(self.model, "named_parameters_with_meta"):
            for _, p, m in self.model.named_parameters_with_meta():
                name = f"parameter_statistics/layers.{m.layer_index}.{m.parameter_name}"
                self.tensor_hook(tensor=p.data, name=name, mode="forward")
                if p.requires_grad:
                    hooks.append(p.register_hook(partial(self.tensor_hook, name=name, mode="backward")))
        else:
            for layer_idx, layer in enumerate(getattr(self.model, "_layers", [])):
                for pname, p in list(layer.named_parameters()) + list(layer.named_buffers()):
                    self.tensor_hook(tensor=p.data, name=f"parameter_statistics/layers.{layer_idx}.{pname}", mode="forward")
        return hooks

    @contextmanager
    def trace(self) -> Iterator[None]:
        hooks = self.register_parameter_hooks()
        fwd = torch.nn.modules.module.register_module_forward_hook(
            lambda module, inp, out: self.activation_hook(module, inp, out, mode="forward"))
        bwd = torch.nn.modules.module.register_module_full_backward_hook(
            lambda module, grad_in, grad_out: self.activation_hook(module, grad_in, grad_out, mode="backward"))
        previous = getattr(self.model, "_tensor_statistics_active", False)
        try:
            self.model._tensor_statistics_active = True  # steps under trace run eagerly
        except Exception:  # noqa: BLE001 - models that refuse attributes are traced all the same
            pass
        try:
            with tensor_tracker.register_hook(self.tensor_hook):
                yield
        finally:
            fwd.remove()
            bwd.remove()
            for h in hooks:
                h.remove()
            try:
                self.model._tensor_statistics_active = previous
            except Exception:  # noqa: BLE001
                pass

    def _module_name(self, module: torch.nn.Module) -> Optional[str]:
        name = self.module_to_name_dict.get(module)
        if name is None:
            for other, mod in self.model.named_modules():
                if mod is module:
                    return other
        return name

    def _global_layer_name(self, name: str) -> tuple[Any, str]:
        """``(global layer index, module path inside the layer)`` of a module path of the model."""
        local = -1
        if "_layers." in name:
            parts = name.split(".")
            local, name = int(parts[1]), ".".join(parts[2:])
        else:
            try:
                local = int(name.split("_")[1])
            except (IndexError, ValueError):
                local = -1
        if local < 0:
            return "index_not_found", name
        coords = getattr(self.model, "_pipe_partition_coordinates", None)
        return (local + coords[0].start if coords else local), name

    def _log(self, value: Any, name: str, mode: str, kind: str) -> None:
        fcts = statistics_fcts_for_name_pattern(self.config.statistics, name)
        if fcts is None:
            return
        if isinstance(value, tuple):
            if len(value) != 1:
                self.logger.warning(f"got a tuple of length {len(value)}, therefore skipping {mode} {kind} hook for {name}")
                return
            value = value[0]
        if not isinstance(value, torch.Tensor):
            self.logger.warning(f"got a value of type {type(value)} but can only handle torch.Tensor, "
                                f"therefore skipping {mode} {kind} hook for {name}")
            return
        with torch.no_grad():
            metrics = {f"{name}_{mode}_{s}": fn(value.detach()) for s, fn in fcts.items()}
        self.logger.log_metrics(metrics=metrics, step=self.context.iterations, to_info=False, to_wandb=False)

    def activation_hook(self, module: torch.nn.Module, input: Any, output: Any,
                        mode: Literal["forward", "backward"] = "forward") -> None:
        name = self._module_name(module)
        if name is None:
            return
        layer_idx, inner = self._global_layer_name(name)
        if self.config.include_module_type:
            full = f"activation_statistics/layers.{layer_idx}.{type(module).__name__}.{inner}"
        else:
            full = f"activation_statistics/layers.{layer_idx}.{inner}"
        self._log(output, full, mode, "activation")

    def tensor_hook(self, tensor: Any, name: str, mode: Literal["forward", "backward"]) -> None:
        self._log(tensor, name, mode, "tensor")
