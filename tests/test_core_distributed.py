"""Engine plumbing on CPU ranks (gloo): batch broadcast, pipeline communicator, data loader resume, schedules, and
how failures of a rank surface (on the host, never on a device)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from scaling_b200.core.nn.pipeline_schedule import PipelineScheduleInference, PipelineScheduleTrain
from scaling_b200.core.nn.pipeline_schedule.simulator import SimulationEngine, illustrate
from tests.utils import dist_launcher

pytestmark = pytest.mark.dist


def _topology(rank, world_size, port, mp=1, pp=1, micro=2, ga=1):
    from scaling_b200.parallel import Topology, TopologyConfig

    cfg = TopologyConfig.from_dict({
        "world_size": world_size, "model_parallel_size": mp, "pipe_parallel_size": pp, "global_rank": rank,
        "local_slot": rank, "micro_batch_size": micro, "gradient_accumulation_steps": ga, "device": "cpu",
        "backend": "gloo"})
    t = Topology(cfg)
    t.initialize_distributed(master_addr="127.0.0.1", master_port=str(port), seed=3)
    return t


# ---------------------------------------------------------------------------------------------- broadcast_data
def _broadcast_worker(rank, world_size, port, device):
    from scaling_b200.core.data import broadcast_data

    t = _topology(rank, world_size, port, mp=2)
    src = [torch.arange(24).reshape(2, 3, 4), torch.tensor([7]), torch.arange(5).reshape(1, 5)]
    got = broadcast_data(src if t.model_parallel_rank == 0 else [None] * 3, dtype=torch.long, topology=t)
    flags = broadcast_data([torch.tensor([True, False, True])] if t.model_parallel_rank == 0 else [None],
                           dtype=torch.bool, topology=t)
    return [None if g is None else (tuple(g.shape), g.flatten().tolist()) for g in got], flags[0].tolist()


def test_broadcast_data_shapes_and_bool():
    r0, r1 = dist_launcher(_broadcast_worker, 2)
    assert r0 == r1
    tensors, flags = r1
    assert tensors[0] == ((2, 3, 4), list(range(24)))
    assert tensors[1] == ((1,), [7]) and tensors[2] == ((1, 5), [0, 1, 2, 3, 4])
    assert flags == [True, False, True]


# ---------------------------------------------------------------------------------------------- pipe communicator
def _pipe_worker(rank, world_size, port, device):
    from scaling_b200.core.nn.parallel_module.communicator import PipeCommunicator

    t = _topology(rank, world_size, port, pp=2)
    comm = PipeCommunicator(local_device=torch.device("cpu"), recv_grads=rank == 0, recv_data=rank == 1,
                            use_continuous_recommunication=True, group=t.pipe_parallel_group,
                            peer_send=1 if rank == 0 else None, peer_recv=0 if rank == 1 else None)
    log = []
    for step, width in enumerate((4, 4, 6)):  # the third payload changes shape: shapes are renegotiated per exchange
        payload = {"h": torch.full((2, width), float(step), requires_grad=True), "meta": ("text", 3, None),
                   "ids": torch.arange(3), "np": np.arange(2)}
        if rank == 0:
            comm.send_data(payload)
            tensors, grads = comm.recv_grad(payload)
            log.append([g.tolist() for g in grads])
        else:
            got = comm.recv_data()
            assert got["meta"] == ("text", 3, None) and got["ids"].tolist() == [0, 1, 2]
            assert got["np"].tolist() == [0, 1] and got["h"].requires_grad
            got["h"].grad = torch.full_like(got["h"], 10.0 + step)
            comm.send_grad(got)
            log.append((tuple(got["h"].shape), got["h"].detach().mean().item()))
    return log


def test_pipe_communicator_moves_pytrees_and_gradients():
    sender, receiver = dist_launcher(_pipe_worker, 2)
    assert receiver == [((2, 4), 0.0), ((2, 4), 1.0), ((2, 6), 2.0)]
    assert [g[0][0][0] for g in sender] == [10.0, 11.0, 12.0]


# ---------------------------------------------------------------------------------------------- data loader
def _loader_worker(rank, world_size, port, device, consumed):
    from scaling_b200.core.data import DataLoader
    from scaling_b200.transformer.data import SyntheticTextDataset

    t = _topology(rank, world_size, port, micro=2)
    ds = SyntheticTextDataset(n_samples=20, sequence_length=4, vocab_size=50, seed=1, low=1)
    loader = DataLoader(seed=1, consumed_samples=consumed, dataset=ds, topology=t, pin_memory=False)
    return [next(loader).token_ids.tolist() for _ in range(4)]


def test_dataloader_resumes_and_shards_by_data_parallel_rank():
    fresh = dist_launcher(_loader_worker, 2, consumed=0)
    resumed = dist_launcher(_loader_worker, 2, consumed=8)  # two global steps of 2 ranks x 2 samples
    for rank in range(2):
        assert fresh[rank][2:] == resumed[rank][:2]
    rows0 = {tuple(r) for batch in fresh[0] for r in batch}
    rows1 = {tuple(r) for batch in fresh[1] for r in batch}
    assert not rows0 & rows1  # the ranks read disjoint samples


# ---------------------------------------------------------------------------------------------- schedules (no ranks)
@pytest.mark.parametrize("pp", [1, 2, 7])
@pytest.mark.parametrize("ga", [1, 2, 7, 16, 32])
def test_schedules_simulate_without_deadlock(pp, ga):
    out = illustrate(PipelineScheduleTrain, ga, pp)
    assert out["steps"] and 0.0 <= out["pct_idling_total"] < 1.0
    engine = SimulationEngine(PipelineScheduleTrain, ga, pp)
    engine.simulate()
    summary = engine.summarize()
    assert summary["total_time"] > 0
    infer = illustrate(PipelineScheduleInference, ga, pp)
    assert infer["steps"]


def test_one_forward_one_backward_bubble():
    out = illustrate(PipelineScheduleTrain, 4, 2)
    assert len(out["steps"]) == 29 and out["pct_idling_total"] == pytest.approx(0.172, abs=1e-3)
    # more micro batches amortise the bubble
    assert illustrate(PipelineScheduleTrain, 32, 2)["pct_idling_total"] < out["pct_idling_total"]


# ---------------------------------------------------------------------------------------------- failures on the host
def _failing_worker(rank, world_size, port, device):
    t = _topology(rank, world_size, port)
    if rank == 1:
        raise RuntimeError("injected failure on rank 1")
    return t.data_parallel_rank


def test_an_exception_on_one_rank_is_reported_with_its_traceback():
    with pytest.raises(AssertionError, match="injected failure on rank 1"):
        dist_launcher(_failing_worker, 2)


def _overflow_worker(rank, world_size, port, device):
    """A non-finite gradient on one rank makes every rank skip the step (fp16-style loss scaling) or raise."""
    from scaling_b200.core.optimizer import (LearningRateSchedulerConfig, LossScalerConfig, Optimizer, OptimizerConfig,
                                             OptimizerParamGroup, OptimizerParamGroupConfig)
    from scaling_b200.core.nn.parameter_meta import CoreParameterMeta

    t = _topology(rank, world_size, port)
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.ones(8))
    CoreParameterMeta.register_on_parameter(p, is_model_parallel=False, layer_index=0, parameter_name="w")
    group = OptimizerParamGroup([("w", p, p.core_parameter_meta)], OptimizerParamGroupConfig(
        name="g", weight_decay=0.0, learning_rate_scheduler=LearningRateSchedulerConfig(learning_rate=0.1)))
    opt = Optimizer(OptimizerConfig(zero=False, loss_scaler=LossScalerConfig(enable=True, initial_scale=4.0, hysteresis=1)),
                    [group], t)
    before = p.detach().clone()
    p.grad.fill_(float("inf") if rank == 1 else 1.0)
    out = opt.step()
    return out.overflow, out.current_loss_scale, torch.equal(p.detach(), before)


def test_overflow_on_one_rank_skips_the_step_everywhere():
    results = dist_launcher(_overflow_worker, 2)
    assert results[0] == results[1] == (True, 2.0, True)


def _added_parameter_worker(rank, world_size, port, device, directory=None):
    """Resume with a parameter that the checkpoint does not know: the restored ones continue their bias correction,
    the new one starts its own, exactly as ``torch.optim.AdamW`` does with one ``step`` per parameter."""
    from scaling_b200.core.optimizer import (LearningRateSchedulerConfig, Optimizer, OptimizerConfig,
                                             OptimizerParamGroup, OptimizerParamGroupConfig)
    from scaling_b200.core.nn.parameter_meta import CoreParameterMeta

    t = _topology(rank, world_size, port)
    zero = world_size > 1

    def build(names):
        torch.manual_seed(3)
        params = []
        for n in names:
            i = "abc".index(n)
            p = torch.nn.Parameter(torch.randn(70 + 10 * i))
            CoreParameterMeta.register_on_parameter(p, is_model_parallel=False, layer_index=i, parameter_name=n)
            params.append((n, p, p.core_parameter_meta))
        group = OptimizerParamGroup(params, OptimizerParamGroupConfig(
            name="g", weight_decay=0.01, learning_rate_scheduler=LearningRateSchedulerConfig(
                learning_rate=0.01, learning_rate_decay_style="constant")))
        opt = Optimizer(OptimizerConfig(zero=zero, beta1=0.9, beta2=0.95, eps=1e-8, gradient_clipping=0.0), [group], t)
        return [p for _, p, _ in params], opt

    def grads(step, params):
        g = torch.Generator().manual_seed(100 + step)
        for p in params:
            p.grad.copy_(torch.randn(p.shape, generator=g))

    old, opt = build(["a", "b"])
    oracle = [torch.nn.Parameter(p.detach().clone()) for p in old]
    ref = torch.optim.AdamW(oracle, lr=0.01, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    for step in range(6):
        grads(step, old)
        for o, p in zip(oracle, old):
            o.grad = p.grad.detach().clone()
        opt.step()
        ref.step()
    first = max((o.detach() - p.detach()).abs().max().item() for o, p in zip(oracle, old))
    opt.save_checkpoint(directory)
    torch.distributed.barrier()

    new, opt2 = build(["a", "c", "b"])  # the new parameter sits between the restored ones in the flat buffer
    opt2.load_checkpoint(directory)
    added = torch.nn.Parameter(new[1].detach().clone())
    ref_added = torch.optim.AdamW([added], lr=0.01, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    ages = [r[2] for r in opt2.parameter_groups[0].step_ranges]
    errs = []
    for step in range(6, 9):
        grads(step, new)
        for o, p in zip(oracle + [added], [new[0], new[2], new[1]]):
            o.grad = p.grad.detach().clone()
        opt2.step()
        ref.step()
        ref_added.step()
        errs.append(max((o.detach() - p.detach()).abs().max().item()
                        for o, p in zip(oracle + [added], [new[0], new[2], new[1]])))
    return ages, opt2.adam_steps, max(errs + [first])


@pytest.mark.parametrize("world_size", [1, 2])
def test_a_parameter_added_at_resume_counts_its_own_adam_steps(tmp_path: Path, world_size):
    results = dist_launcher(_added_parameter_worker, world_size, directory=str(tmp_path))
    for ages, adam_steps, err in results:
        assert ages == [0, 6, 0] and adam_steps == 9
        assert err < 1e-6


def _pattern_on_another_stage_worker(rank, world_size, port, device):
    """A finetuning pattern may match parameters of another pipeline stage only; it fails if it matches on no rank."""
    from scaling_b200.transformer.context.config import TrainingGroupConfig
    from scaling_b200.transformer.model.model import _extract_parameters

    _topology(rank, world_size, port)
    mine = [("stage0.image_encoder.w", torch.nn.Parameter(torch.zeros(1)), None)] if rank == 0 else \
        [("stage1.summarization.w", torch.nn.Parameter(torch.zeros(1)), None)]
    group = [TrainingGroupConfig(group_name="g", parameters_include=["summarization", "image_encoder"])]
    (members, _), = _extract_parameters(group, mine, True)
    try:
        _extract_parameters([TrainingGroupConfig(group_name="g", parameters_include=["summarization", "nowhere"])],
                            mine, True)
        error = None
    except ValueError as e:
        error = str(e)
    return [n for n, _, _ in members], error


def test_finetuning_patterns_are_matched_over_all_ranks():
    results = dist_launcher(_pattern_on_another_stage_worker, 2)
    assert results[0][0] == ["stage0.image_encoder.w"] and results[1][0] == ["stage1.summarization.w"]
    assert all("Unmatched finetunable parameters: {'nowhere'}" in r[1] for r in results)


def _collective_forms_worker(rank, world_size, port, device):
    """``all_concat`` / ``all_shard`` with an explicit dimension and the gather over tokens with and without the
    gradient reduction, called the way src/scaling/core/nn/linear/utils.py:195-252 declares them."""
    from scaling_b200.parallel.collectives import all_concat, all_shard, gather_from_sequence_parallel_region

    t = _topology(rank, world_size, port, mp=2)
    torch.manual_seed(1)
    full = torch.randn(2, 4, 6)
    mine = full[:, rank * 2:(rank + 1) * 2].clone().requires_grad_()
    gathered = all_concat(mine, 1, t)
    ok = torch.equal(gathered, full) and torch.equal(all_concat(input_tensor=mine, dim=1, topology=t), full)
    (gathered * full).sum().backward()
    ok &= torch.equal(mine.grad, full[:, rank * 2:(rank + 1) * 2])
    ok &= torch.equal(all_shard(full, 1, t), full[:, rank * 2:(rank + 1) * 2])
    ok &= torch.equal(all_shard(full, t), full[..., rank * 3:(rank + 1) * 3])
    grads = []
    for reduce_grad in (True, False):
        tokens = full[:, rank * 2:(rank + 1) * 2].clone().requires_grad_()
        out = gather_from_sequence_parallel_region(tokens, t, tensor_parallel_output_grad=reduce_grad)
        ok &= out.shape == full.shape
        (out * (rank + 1.0)).sum().backward()
        grads.append(float(tokens.grad[0, 0, 0]))
    return bool(ok), grads


def test_collectives_accept_the_dimension_and_gradient_forms():
    for rank, (ok, grads) in enumerate(dist_launcher(_collective_forms_worker, 2)):
        assert ok
        assert grads == [3.0, rank + 1.0]  # summed over both ranks' consumers, or this rank's own gradient only
