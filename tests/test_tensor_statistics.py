"""Tensor statistics recorder: metric names, pattern selection, hook removal."""

import torch

from scaling_b200.core.logging.tensor_statistics_recorder import (TENSOR_STATISTICS_FUNCTIONS, TensorStatistics,
                                                                  TensorStatisticsRecorder,
                                                                  TensorStatisticsRecorderConfig,
                                                                  statistics_fcts_for_name_pattern, tensor_tracker)


class _Logger:
    def __init__(self):
        self.metrics = {}

    def log_metrics(self, metrics, step, to_info=True, to_wandb=True):
        self.metrics.update(metrics)

    def warning(self, *_):
        pass


class _Context:
    iterations = 7


class _Model(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self._layers = torch.nn.ModuleList([torch.nn.Linear(4, 4), torch.nn.Linear(4, 2)])

    def forward(self, x):
        h = self._layers[0](x)
        tensor_tracker.trace_tensor(h, "hidden")
        return self._layers[1](h)


def test_every_statistic_is_computable():
    assert len(TensorStatistics) == 33 and set(TENSOR_STATISTICS_FUNCTIONS) == set(TensorStatistics)
    x = torch.softmax(torch.randn(16, 32), dim=-1)
    for stat, fn in TENSOR_STATISTICS_FUNCTIONS.items():
        assert isinstance(fn(x), float), stat
    assert TENSOR_STATISTICS_FUNCTIONS[TensorStatistics.PCT_ZERO](torch.tensor([0.0, 1.0])) == 0.5
    assert TENSOR_STATISTICS_FUNCTIONS[TensorStatistics.QUANTILE_75](torch.arange(5.0)) == 3.0


def test_pattern_selection_first_match_wins():
    cfg = [("*weight*", [TensorStatistics.MAX]), ("*", [TensorStatistics.MEAN, TensorStatistics.STD])]
    assert list(statistics_fcts_for_name_pattern(cfg, "parameter_statistics/layers.0.weight")) == ["max"]
    assert list(statistics_fcts_for_name_pattern(cfg, "activation_statistics/layers.1.x")) == ["mean", "std"]
    assert statistics_fcts_for_name_pattern([("a*", [TensorStatistics.MAX])], "b") is None


def test_trace_records_activations_parameters_and_tracked_tensors():
    model, log = _Model(), _Logger()
    cfg = TensorStatisticsRecorderConfig(statistics=[("*", [TensorStatistics.MEAN, TensorStatistics.ABS_MAX])])
    rec = TensorStatisticsRecorder(cfg, _Context(), model, logger=log)
    with rec.trace():
        model(torch.randn(3, 4)).sum().backward()
    names = set(log.metrics)
    assert "activation_statistics/layers.0._forward_mean" in names
    assert "activation_statistics/layers.1._backward_abs_max" in names
    assert "parameter_statistics/layers.0.weight_forward_mean" in names
    assert "parameter_statistics/layers.1.bias_forward_mean" in names
    assert "tensor_statistics/counter.0.hidden_forward_mean" in names
    assert "tensor_statistics/counter.0.hidden_backward_mean" in names
    # everything is unhooked afterwards
    log.metrics.clear()
    model(torch.randn(3, 4)).sum().backward()
    assert not log.metrics and not tensor_tracker.hooks
