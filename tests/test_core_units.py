"""Unit tests of the engine's host-side pieces (no GPU, no process groups)."""

import errno
import json
from pathlib import Path
from typing import Optional

import pytest
import torch
from pydantic import Field, ValidationError

from scaling_b200.core.config import BaseConfig
from scaling_b200.core.data.file_handles import FileHandle, RetryableException
from scaling_b200.core.nn.parallel_module.pipeline_partitioning import (PipePartitionCoordinates, balanced_boundaries,
                                                                        pipe_partition_from_indices,
                                                                        pipe_partition_uniform)
from scaling_b200.core.optimizer import (LearningRateDecayStyle, LearningRateScheduler, LearningRateSchedulerConfig,
                                         LossScaler, LossScalerConfig)
from scaling_b200.core.runner import RunnerConfig
from scaling_b200.core.runner.runner import hosts_str_to_resource_pool, parse_host
from scaling_b200.parallel import TopologyConfig


# ---------------------------------------------------------------------------------------------- config
class _Inner(BaseConfig):
    width: int = Field(4, description="inner width")


class _Outer(BaseConfig):
    name: str = Field("x", description="a name")
    inner: _Inner = Field(_Inner(), description="nested settings")
    items: Optional[list[int]] = Field(None, description="numbers")


def test_config_is_frozen_and_forbids_unknown_keys():
    c = _Outer.from_dict({"name": "a", "inner": {"width": 8}})
    assert c.inner.width == 8
    with pytest.raises(ValidationError):
        c.name = "b"
    with pytest.raises(ValidationError):
        _Outer.from_dict({"nam": "typo"})


def test_config_round_trips_and_overwrites(tmp_path: Path):
    c = _Outer.from_dict({"name": "a", "items": [1, 2]}, overwrite_values={"inner": {"width": 16}})
    assert c.inner.width == 16 and c.items == [1, 2]
    assert _Outer.from_str(c.as_str()) == c
    assert json.loads(c.as_str())["inner"]["width"] == 16
    c.save(tmp_path / "c.yml")
    assert _Outer.from_yaml(tmp_path / "c.yml") == c
    assert _Outer.from_yaml(tmp_path / "c.yml", overwrite_values={"name": "z"}).name == "z"


def test_config_template_lists_every_field_with_its_description(tmp_path: Path):
    text = _Outer.get_template_str()
    for needle in ("name", "a name", "inner", "width", "inner width", "items"):
        assert needle in text
    _Outer.save_template(tmp_path / "t.yml")
    assert (tmp_path / "t.yml").read_text()


# ---------------------------------------------------------------------------------------------- topology
@pytest.mark.parametrize("given,expected", [
    (dict(world_size=8, model_parallel_size=2, pipe_parallel_size=2), dict(data_parallel_size=2)),
    (dict(world_size=8, model_parallel_size=2, data_parallel_size=4), dict(pipe_parallel_size=1)),
    (dict(model_parallel_size=2, pipe_parallel_size=2, data_parallel_size=3), dict(world_size=12)),
    (dict(world_size=4, pipe_parallel_size=2, data_parallel_size=2), dict(model_parallel_size=1)),
])
def test_topology_infers_the_missing_parallel_size(given, expected):
    t = TopologyConfig.from_dict(dict(given, micro_batch_size=2, gradient_accumulation_steps=1))
    for k, v in expected.items():
        assert getattr(t, k) == v
    assert t.world_size == t.model_parallel_size * t.pipe_parallel_size * t.data_parallel_size


def test_topology_batch_triple():
    base = dict(world_size=4, model_parallel_size=1, pipe_parallel_size=1, data_parallel_size=4)
    t = TopologyConfig.from_dict(dict(base, micro_batch_size=2, gradient_accumulation_steps=3))
    assert t.global_batch_size == 24
    t = TopologyConfig.from_dict(dict(base, global_batch_size=32, micro_batch_size=2))
    assert t.gradient_accumulation_steps == 4
    t = TopologyConfig.from_dict(dict(base, global_batch_size=32, gradient_accumulation_steps=2))
    assert t.micro_batch_size == 4
    with pytest.raises((ValidationError, AssertionError, ValueError)):
        TopologyConfig.from_dict(dict(base, global_batch_size=30, micro_batch_size=2, gradient_accumulation_steps=2))
    with pytest.raises((ValidationError, AssertionError, ValueError)):
        TopologyConfig.from_dict(dict(world_size=8, model_parallel_size=3, pipe_parallel_size=1, micro_batch_size=1,
                                      gradient_accumulation_steps=1))


# ---------------------------------------------------------------------------------------------- learning rate
def test_learning_rate_warmup_and_decay_styles():
    def sched(style, **kw):
        return LearningRateScheduler(LearningRateSchedulerConfig(
            learning_rate=1.0, learning_rate_minimum=0.1, learning_rate_decay_style=style,
            learning_rate_decay_iters=100, learning_rate_warmup_steps=10, **kw))

    cos = sched(LearningRateDecayStyle.COSINE)
    assert cos.get_lr(0) == pytest.approx(0.0)
    assert cos.get_lr(5) == pytest.approx(0.5)
    assert cos.get_lr(10) == pytest.approx(1.0)
    assert cos.get_lr(55) == pytest.approx(0.55, abs=1e-6)  # halfway through the cosine
    assert cos.get_lr(100) == pytest.approx(0.1)
    assert cos.get_lr(10_000) == pytest.approx(0.1)
    lin = sched(LearningRateDecayStyle.LINEAR)
    assert lin.get_lr(55) == pytest.approx(0.55, abs=1e-6)
    const = sched(LearningRateDecayStyle.CONSTANT)
    assert const.get_lr(50) == pytest.approx(1.0)
    lrs = [cos.get_lr(i) for i in range(10, 101)]
    assert all(a >= b for a, b in zip(lrs, lrs[1:]))  # monotone after warm-up


# ---------------------------------------------------------------------------------------------- loss scaler
def test_loss_scaler_state_machine():
    s = LossScaler(LossScalerConfig(enable=True, initial_scale=2.0 ** 8, window=3, hysteresis=2, factor=2.0, min_scale=1.0))
    assert s.scale_loss(torch.tensor(1.0)).item() == 256.0
    out = s.step(overflow=True)  # first overflow only spends hysteresis
    assert out.overflow and out.current_loss_scale == 256.0
    out = s.step(overflow=True)  # second one halves the scale
    assert out.current_loss_scale == 128.0
    for _ in range(3):
        out = s.step(overflow=False)
    assert out.current_loss_scale == 128.0 and out.no_overflow_steps == 3
    out = s.step(overflow=False)  # the step after a full clean window doubles the scale
    assert out.current_loss_scale == 256.0
    state = s.state_dict()
    s2 = LossScaler(LossScalerConfig(enable=True))
    s2.load_state_dict(state)
    assert s2.current_scale == s.current_scale
    off = LossScaler(LossScalerConfig(enable=False))
    assert off.scale_loss(torch.tensor(3.0)).item() == 3.0
    assert off.step(False).current_loss_scale is None


# ---------------------------------------------------------------------------------------------- retryable reads
class _Flaky:
    def __init__(self, failures: int, exc: BaseException):
        self.failures, self.exc, self.calls = failures, exc, 0

    def __call__(self, f):
        self.calls += 1
        if self.calls <= self.failures:
            raise self.exc
        return f.read()


def test_file_handle_retries_stale_handles(tmp_path: Path, monkeypatch):
    monkeypatch.setattr(FileHandle, "sleep", staticmethod(lambda _s: None))  # no real back-off in the test
    path = tmp_path / "data.bin"
    path.write_bytes(b"payload")
    handle = FileHandle(path)
    flaky = _Flaky(2, OSError(errno.ESTALE, "stale file handle"))
    assert handle.retry_operation(flaky) == b"payload" and flaky.calls == 3
    flaky = _Flaky(1, RetryableException("try again"))
    assert handle.retry_operation(flaky) == b"payload"
    with pytest.raises(OSError):  # other errors are not retried
        handle.retry_operation(_Flaky(1, OSError(errno.EACCES, "denied")))
    always = _Flaky(99, OSError(errno.ESTALE, "stale"))
    with pytest.raises(Exception, match="even after 4 retries"):
        handle.retry_operation(always, max_attempts=4)
    assert always.calls == 4
    handle.close()


# ---------------------------------------------------------------------------------------------- partitioning
@pytest.mark.parametrize("items,parts", [(10, 3), (4, 4), (7, 2), (16, 5), (3, 1)])
def test_uniform_partition_covers_all_layers(items, parts):
    coords = pipe_partition_uniform(items, parts)
    assert len(coords) == parts and coords[0].start == 0 and coords[-1].end == items
    assert all(a.end == b.start for a, b in zip(coords, coords[1:]))
    lengths = [c.length for c in coords]
    assert max(lengths) - min(lengths) <= 1 and lengths == sorted(lengths, reverse=True)  # remainder goes first


def test_manual_and_balanced_partitions():
    assert pipe_partition_from_indices([0, 3, 5, 9], num_layers=9) == [
        PipePartitionCoordinates(0, 3), PipePartitionCoordinates(3, 5), PipePartitionCoordinates(5, 9)]
    with pytest.raises(ValueError):
        pipe_partition_from_indices([0, 3, 5], num_layers=9)  # the last boundary has to be the layer count
    bounds = balanced_boundaries([10, 1, 1, 1, 1, 10], 3)
    assert bounds[0] == 0 and bounds[-1] == 6 and len(bounds) == 4
    loads = [sum([10, 1, 1, 1, 1, 10][a:b]) for a, b in zip(bounds, bounds[1:])]
    assert max(loads) == 10  # the optimum: no stage heavier than the heaviest single layer


# ---------------------------------------------------------------------------------------------- runner
def test_runner_parses_hosts():
    cfg = RunnerConfig(default_gpu_count=8)
    assert parse_host(cfg, "node-1 slots=4") == ("node-1", [0, 1, 2, 3])
    assert parse_host(cfg, "node-2 slots=0,2,5") == ("node-2", [0, 2, 5])
    assert parse_host(cfg, "node-3") == ("node-3", list(range(8)))
    pool = hosts_str_to_resource_pool(cfg, ["a slots=2", "b slots=1"])
    assert list(pool.items()) == [("a", [0, 1]), ("b", [0])]
    with pytest.raises((ValueError, AssertionError)):
        hosts_str_to_resource_pool(cfg, ["a slots=2", "a slots=2"])


# ---------------------------------------------------------------------------------------------- attention ranges
def test_document_ranges_have_to_cover_every_token():
    from scaling_b200.ops.attention_kernel import _check_ranges

    ok = torch.zeros(8, dtype=torch.int32)
    _check_ranges(ok, ok, 8)
    with pytest.raises(ValueError, match="cover 4"):
        _check_ranges(ok[:4], ok[:4], 8)  # e.g. ranges of one sequence-parallel shard handed to the gathered sequence
    with pytest.raises(ValueError):
        _check_ranges(ok.long(), ok.long(), 8)


def test_document_ranges_follow_the_position_ids_not_the_local_activations():
    from scaling_b200.transformer.data.utils import document_ranges_from_padded

    padded = torch.tensor([0, 3, 8, -1, -1])
    start, end = document_ranges_from_padded(padded, 8)
    assert start.tolist() == [0, 0, 0, 3, 3, 3, 3, 3] and end.tolist() == [3, 3, 3, 8, 8, 8, 8, 8]


# ---------------------------------------------------------------------------------------------- benchmark layouts
@pytest.mark.parametrize("config,gpus,expected", [
    ("125m", 8, dict(mp=1, pp=1, dp=8, ga=1)),
    ("7b", 8, dict(mp=4, pp=1, dp=2, ga=32)),
    ("7b", 2, dict(mp=2, pp=1, dp=1, ga=64)),
    ("7b_lora", 8, dict(mp=8, pp=1, dp=1, ga=32)),
    ("13b", 8, dict(mp=2, pp=2, dp=2, ga=16)),
    ("13b", 2, dict(mp=2, pp=1, dp=1, ga=32)),
])
def test_benchmark_layouts_fit_the_gpus(config, gpus, expected):
    import argparse
    import importlib.util
    from pathlib import Path as _P

    spec = importlib.util.spec_from_file_location("bench_module", _P(__file__).resolve().parent.parent / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    lay = bench.layout(argparse.Namespace(config=config, grad_accum=None, layers=None, sequence_parallel=False), gpus)
    assert {k: lay[k] for k in expected} == expected
    assert lay["mp"] * lay["pp"] * lay["dp"] == gpus
    assert bench.model_flops_per_token(lay["arch"], True) > bench.model_flops_per_token(lay["arch"], False) > 0


# ---------------------------------------------------------------------------------------------- 1F1B order
def test_one_forward_one_backward_instruction_order():
    from scaling_b200.core.nn.pipeline_schedule import PipelineScheduleTrain
    from scaling_b200.parallel import Topology

    def order(stage):
        cfg = TopologyConfig.from_dict({"world_size": 2, "model_parallel_size": 1, "pipe_parallel_size": 2,
                                        "global_rank": stage, "micro_batch_size": 1, "gradient_accumulation_steps": 4,
                                        "device": "cpu", "backend": "gloo"})
        short = {"LoadMicroBatch": "Load", "ForwardPass": "F", "BackwardPass": "B", "SendActivation": "SendA",
                 "RecvActivation": "RecvA", "SendGrad": "SendG", "RecvGrad": "RecvG", "Loss": "Loss",
                 "ReduceTiedGrads": "ReduceTied", "OptimizerStep": "OptStep"}
        return [(short[i.name], i.micro_batch_id, i.buffer_id) for i in PipelineScheduleTrain(Topology(cfg)).instructions()]

    names0 = [f"{n}{'' if m is None else m}" for n, m, _ in order(0)]
    assert names0 == ("Load0 F0 SendA0 Load1 F1 SendA1 RecvG0 B0 Load2 F2 SendA2 RecvG1 B1 Load3 F3 SendA3 RecvG2 B2 "
                      "RecvG3 B3 ReduceTied OptStep").split()
    names1 = [f"{n}{'' if m is None else m}" for n, m, _ in order(1)]
    assert names1 == ("RecvA0 Load0 F0 Loss0 B0 RecvA1 SendG0 Load1 F1 Loss1 B1 RecvA2 SendG1 Load2 F2 Loss2 B2 "
                      "RecvA3 SendG2 Load3 F3 Loss3 B3 SendG3 ReduceTied OptStep").split()
    # buffers: micro batch modulo max(2, min(stages - stage + 1, micro batches))
    assert {m: b for n, m, b in order(0) if n == "Load"} == {0: 0, 1: 1, 2: 2, 3: 0}
    assert {m: b for n, m, b in order(1) if n == "RecvA"} == {0: 0, 1: 1, 2: 0, 3: 1}


# ---------------------------------------------------------------------------------------------- public names
def test_public_names_of_the_two_packages():
    import scaling_b200.core as core
    import scaling_b200.transformer as transformer

    core_names = """BaseConfig BaseContext BaseContextGeneric DeterminedBaseContext BaseBlendedDataset BaseDataset
        BaseDatasetBatch BaseDatasetItem BaseLayerIO BlendedDatasetConfig DataLoader FileDataset MemoryMapDataset
        MemoryMapDatasetBuilder broadcast_data ActivationFunction BaseLayer ColumnParallelLinear CoreParameterMeta
        LayerNorm LayerNormConfig LayerNormOptimizationType LayerSpec LoRaConfig LoRAModuleType MaskedSoftmax
        MaskedSoftmaxConfig MaskedSoftmaxKernel NormType ParallelLoRa ParallelMLP ParallelModule ParallelSelfAttention
        ParallelSwiGLUMLP PipelineScheduleInference PipelineScheduleTrain PipePartitionCoordinates
        RelativePositionEmbeddingType RMSNorm RotaryConfig RotaryEmbedding RotaryEmbeddingComplex RowParallelLinear
        TiedLayerSpec VocabParallelEmbedding get_activation_function get_norm pipe_partition_uniform BaseOptimizer
        LearningRateDecayStyle LearningRateScheduler LearningRateSchedulerConfig LossScaler LossScalerConfig Optimizer
        OptimizerConfig OptimizerParamGroup OptimizerParamGroupConfig Profiler ProfilerConfig SynchronizedTimer
        RunnerConfig RunnerDockerConfig RunnerType runner_main PipePartitionMethod Topology TopologyConfig BaseTrainer
        DeterminedBaseTrainer TrainerConfig""".split()
    assert [n for n in core_names if not hasattr(core, n)] == []
    transformer_names = """TransformerConfig TransformerContext EmbeddingDataset EmbeddingBlendedDataset
        FinetuningChatDataset FinetuningChatBlendedDataset FinetuningTextDataset FinetuningTextBlendedDataset
        LegacyBlendedDataset TextDataset TextBlendedDataset TextDatasetItem TransformerLayerIO TransformerParallelModule
        init_model init_optimizer""".split()
    assert [n for n in transformer_names if not hasattr(transformer, n)] == []
    from scaling_b200.core.nn.parallel_module import EvaluationStepOutput, TrainStepOutput
    from scaling_b200.core.nn.parallel_module.inference_module import InferenceModule, RecorderSetting  # noqa: F401
    from scaling_b200.core.runner.launch_config import LaunchConfig  # noqa: F401
    from scaling_b200.core.utils.port import find_free_port  # noqa: F401
    from scaling_b200.transformer.inference import TransformerInferenceModule  # noqa: F401
    from scaling_b200.transformer.model.losses import create_loss_function  # noqa: F401
    from scaling_b200.transformer.model.model import get_transformer_layer_specs  # noqa: F401
    from scaling_b200.transformer.tokenizer import Tokenizer, load_tokenizers  # noqa: F401
    from scaling_b200.transformer.train import main  # noqa: F401

    assert TrainStepOutput._fields == ("loss", "metrics", "global_grad_norm", "global_grad_norm_clipped",
                                       "learning_rates", "overflow", "no_overflow_steps", "current_loss_scale",
                                       "step_duration", "debug_dict")
    assert EvaluationStepOutput._fields == ("loss", "metrics", "step_duration")


# ---------------------------------------------------------------------------------------------- u-muP multipliers
def test_unit_scaled_multipliers_and_residual_scales():
    from scaling_b200.core.nn.parameter_meta import UMUP_WEIGHT_TYPE, CoreParameterMeta, UMuPParameterMeta
    from scaling_b200.core.nn.umup import UMuParametrization as U

    def meta(shape, kind, parallel_dim=None, on_residual=False):
        m = CoreParameterMeta(local_shape=shape, is_model_parallel=parallel_dim is not None,
                              model_parallel_dimension=parallel_dim)
        m.umup_meta = UMuPParameterMeta(weight_type=kind, on_residual=on_residual)
        return m

    B, depth = 4096, 16
    assert U.get_parameter_multipliers(meta((64,), UMUP_WEIGHT_TYPE.NORM), 1, B, depth) == (1.0, 1.0, B ** -0.5, 1.0)
    # column-parallel hidden weight [out / 2, in]: fan-in is the full input width
    f, b, g, lr = U.get_parameter_multipliers(meta((32, 256), UMUP_WEIGHT_TYPE.HIDDEN_WEIGHT, 0, True), 2, B, depth)
    assert (f, b, g) == (256 ** -0.5, 256 ** -0.5, B ** -0.5) and lr == pytest.approx(256 ** -0.5 * depth ** -0.5)
    # row-parallel output weight [out, in / 2]: fan-in counts every rank's slice
    f, b, g, lr = U.get_parameter_multipliers(meta((100, 128), UMUP_WEIGHT_TYPE.OUTPUT_WEIGHT, 1), 2, B, depth)
    assert (f, b, g, lr) == (1.0 / 256, 100 ** -0.5, B ** -0.5, 1.0)
    f, b, g, lr = U.get_parameter_multipliers(meta((500, 64), UMUP_WEIGHT_TYPE.INPUT_EMBEDDING, 0), 2, B, depth)
    assert (f, b, lr) == (1.0, 1.0, 64 ** -0.5) and g == pytest.approx((B / 1000) ** -0.5)
    # residual scales keep unit variance: a^2 + b^2 = 1, later branches weigh less under pre-norm
    mults = U.get_umup_transformer_residual_mults(1.0, 1.0, num_layers=2)
    assert mults == [1.0, 1.0, 1.0, 1.0]
    scales = [U.get_umup_residual_scales(mults, i, pre_norm=True, depth=4) for i in range(4)]
    assert all(a * a + b * b == pytest.approx(1.0) for a, b in scales)
    assert [a for a, _ in scales] == sorted((a for a, _ in scales), reverse=True)
    mult, out_scale = U.get_umup_cross_entropy_scales(1.0, 1000)
    assert mult == 1.0 and out_scale == pytest.approx(1000 / 999 ** 0.5)
    att, _ = U.get_umup_attention_scales(head_dim=64, sequence_length=2048, mult=1.0, dropout_p=0.0)
    assert att == 1.0 / 64


# ---------------------------------------------------------------------------------------------- Determined glue
def test_hyper_parameters_become_config_overrides():
    from scaling_b200.transformer.train_determined import hparams_to_overrides

    hp = {"learning_rate": 3e-4, "target_train_tokens": 2_000_000, "warmup_tokens": 200_000, "sequence_length": 1000,
          "global_batch_size": 20, "kernel": "flash_attention", "sequence_parallel": True}
    out = hparams_to_overrides(hp, {"trainer": {"seed": 7}})
    assert out["trainer"] == {"seed": 7, "train_iterations": 100}
    assert out["learning_rate_scheduler"] == {"learning_rate": 3e-4, "learning_rate_warmup_steps": 10}
    assert out["transformer_architecture"]["masked_softmax"] == {"kernel": "flash_attention"}
    assert out["topology"]["sequence_parallel"] is True
    # a restarted single run carries its whole layout, which replaces the search space
    assert hparams_to_overrides({"layout": {"learning_rate": 1.0}, "learning_rate": 2.0})["learning_rate_scheduler"] == {
        "learning_rate": 1.0}
    assert hparams_to_overrides(None, {"a": 1}) == {"a": 1}


def test_training_groups_select_parameters_by_pattern():
    """Include / exclude patterns pick the members of an optimizer group; a pattern that matches nothing, a parameter
    claimed by two groups and a parameter left without a group are errors (the last one can be allowed)."""
    import pytest
    import torch

    from scaling_b200.transformer.context.config import TrainingGroupConfig
    from scaling_b200.transformer.model.model import _extract_parameters

    def named(*names):
        return [(n, torch.nn.Parameter(torch.zeros(1)), None) for n in names]

    params = named("layers.1.adapter_x.weight", "layers.1.adapter_x.bias", "layers.1.mlp.weight", "image_encoder.baz")
    pick = [TrainingGroupConfig(group_name="g", parameters_include=["adapter_x", "image_encoder"],
                                parameters_exclude=[r"\.bias$"])]
    (members, group), = _extract_parameters(pick, params, allow_missing_params_in_optimizer=True)
    assert [n for n, _, _ in members] == ["layers.1.adapter_x.weight", "image_encoder.baz"] and group.group_name == "g"
    with pytest.raises(ValueError, match="not added to any optimizer group"):
        _extract_parameters(pick, params, allow_missing_params_in_optimizer=False)
    with pytest.raises(ValueError, match=r"Unmatched finetunable parameters: \{'summarization'\}"):
        _extract_parameters([TrainingGroupConfig(group_name="g", parameters_include=["adapter_x", "summarization"])],
                            params, True)
    overlap = [TrainingGroupConfig(group_name="a", parameters_include=["adapter_x"]),
               TrainingGroupConfig(group_name="b", parameters_include=[r"\.bias$"])]
    with pytest.raises(ValueError, match="more then one training_group"):
        _extract_parameters(overlap, params, True)
    everything = _extract_parameters([TrainingGroupConfig(group_name="all")], params, False)
    assert len(everything[0][0]) == 4


def test_logger_rank_filter_sinks_and_wandb_key(monkeypatch):
    """Metrics sinks default to global rank 0 and otherwise follow the configured rank list; the singleton swaps
    its implementation on ``configure`` / ``configure_determined``; wandb needs a key from the config or the
    environment."""
    import pytest
    from pydantic import ValidationError

    from scaling_b200.core.logging import DeterminedLogger, Logger, LoggerConfig, logger
    from scaling_b200.core.logging.logger_config import check_if_in_rank

    for ranks in ([], None, [0], [42], [36]):
        for rank in (None, 0, 42):
            want = rank is not None and ((ranks is None and rank == 0) or (ranks is not None and rank in ranks))
            assert check_if_in_rank(rank, ranks) == want
    logger.configure(LoggerConfig())
    assert type(logger._impl) is Logger
    logger.configure_determined(LoggerConfig())
    assert type(logger._impl) is DeterminedLogger
    logger.log_metrics({"training/loss": 1.0}, step=1)  # no Determined context: nothing to report to, no error
    logger.configure(LoggerConfig())
    assert type(logger._impl) is Logger

    monkeypatch.setenv("WANDB_API_KEY", "from-env")
    assert LoggerConfig().wandb_api_key == "from-env"
    assert LoggerConfig(wandb_api_key="given").wandb_api_key == "given"
    assert LoggerConfig(use_wandb=True).wandb_api_key == "from-env"
    monkeypatch.setenv("WANDB_API_KEY", "")
    with pytest.raises(ValidationError, match="wandb api key needs to be provided"):
        LoggerConfig(use_wandb=True)
    monkeypatch.delenv("WANDB_API_KEY")
    with pytest.raises(ValidationError):
        LoggerConfig(use_wandb=True, wandb_api_key=None)
    assert LoggerConfig(use_wandb=True, wandb_api_key="k").use_wandb
    assert not LoggerConfig(use_wandb=False, wandb_api_key="").use_wandb


def test_tied_layer_spec_argument_orders_and_rank_groups():
    """``TiedLayerSpec`` takes its three leading arguments by keyword, module class first, or key first; rank groups
    can be returned nested."""
    import torch

    from scaling_b200.core.nn.parallel_module.layer_spec import TiedLayerSpec
    from scaling_b200.parallel import Topology, TopologyConfig

    lin = torch.nn.Linear
    specs = [TiedLayerSpec(lin, "k", ["weight"], 3, 4), TiedLayerSpec("k", ["weight"], lin, in_features=3, out_features=4),
             TiedLayerSpec(module_class=lin, key="k", tied_weight_attributes=["weight"], in_features=3, out_features=4)]
    for s in specs:
        assert s.key == "k" and s.tied_weight_attributes == ["weight"] and s.initialize().weight.shape == (4, 3)
    t = Topology(TopologyConfig.from_dict({"world_size": 8, "model_parallel_size": 2, "pipe_parallel_size": 2,
                                           "data_parallel_size": 2, "global_rank": 0, "micro_batch_size": 1,
                                           "gradient_accumulation_steps": 1, "device": "cpu", "backend": "gloo"}))
    flat = t.get_global_rank_group(pipe_parallel_rank=1)
    nested = t.get_global_rank_group(pipe_parallel_rank=1, flatten=False)
    assert len(flat) == 4 and len(nested) == 1 and len(nested[0]) == 2 and len(nested[0][0]) == 2
    assert [r for d in nested[0] for r in d] == flat
