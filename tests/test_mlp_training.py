"""End-to-end training of the MLP application on CPU ranks (gloo): parallel layouts agree with a
single process, and a resumed run reproduces the loss curve exactly."""

import copy
from pathlib import Path

import pytest

from tests.utils import dist_launcher


def _config(world_size, mp=1, pp=1, zero=False, ga=1, micro=16, iters=10, save_dir=None, load_dir=None,
            save_interval=None, ckpt="disabled", precision="float32"):
    dp = world_size // (mp * pp)
    return {
        "topology": {"world_size": world_size, "model_parallel_size": mp, "pipe_parallel_size": pp,
                     "data_parallel_size": dp, "micro_batch_size": micro // dp if dp > 1 else micro,
                     "gradient_accumulation_steps": ga, "device": "cpu", "backend": "gloo",
                     "activation_checkpointing_type": ckpt},
        "optimizer": {"zero": zero, "gradient_clipping": 1.0},
        "learning_rate_scheduler": {"learning_rate": 1e-3, "learning_rate_decay_style": "constant"},
        "trainer": {"train_iterations": iters, "seed": 7, "save_dir": save_dir, "load_dir": load_dir,
                    "save_interval": save_interval, "assert_checkpoint_loaded": load_dir is not None,
                    "delete_past_optimizer_states": False},
        "architecture": {"n_hidden_layers": 1, "hidden_dim": 64, "precision": precision},
        "data": {"n_samples": 512},
    }


def _run(rank, world_size, port, device, config, save_initial=None):
    from scaling_b200.core.runner import LaunchConfig
    from scaling_b200.core.trainer import BaseTrainer
    from scaling_b200.models.mlp import (MLPConfig, MLPContext, SyntheticClassificationDataset, init_model,
                                         init_optimizer, loss_function, metrics_aggregation_fn)
    from scaling_b200.parallel import Topology

    lc = LaunchConfig(master_port=port, master_addr="127.0.0.1", world_size=world_size, global_rank=rank,
                      local_slot=rank, payload=copy.deepcopy(config))
    cfg = MLPConfig.from_dict(lc.overwrite_config_dict_with_launcher_args(dict(lc.payload)))
    topology = Topology(cfg.topology)
    context = MLPContext(config=cfg, topology=topology)
    context.initialize(master_addr="127.0.0.1", master_port=str(port), seed=cfg.trainer.seed)
    model = init_model(context)
    optimizer = init_optimizer(context, model)
    dataset = SyntheticClassificationDataset(n_samples=cfg.data.n_samples, seed=cfg.trainer.seed) if topology.is_io_rank else None
    trainer = BaseTrainer(config=cfg.trainer, context=context, parallel_module=model, optimizer=optimizer,
                          dataset=dataset, sync_batch_to_model_parallel=SyntheticClassificationDataset.sync_batch_to_model_parallel,
                          loss_function=loss_function, metrics_aggregation_fn=metrics_aggregation_fn)
    if save_initial is not None:
        trainer.save_checkpoint(Path(save_initial))
    metrics = trainer.run_training(return_metrics=True)
    return [m["training/loss"] for m in metrics] if metrics else None


def _losses(world_size, save_initial=None, **kw):
    res = dist_launcher(_run, world_size, config=_config(world_size, **kw), save_initial=save_initial)
    return res[0]


@pytest.mark.dist
def test_layouts_agree_with_single_process(tmp_path: Path):
    init = str(tmp_path / "init")
    base = _losses(1, save_initial=init)
    assert base[-1] < base[0]
    for kw in (dict(world_size=2, mp=2), dict(world_size=2, pp=2, ga=2, micro=8), dict(world_size=2, zero=True),
               dict(world_size=2), dict(world_size=1, ga=4, micro=4), dict(world_size=1, ckpt="every_layer")):
        ws = kw.pop("world_size")
        got = _losses(ws, load_dir=init, **kw)
        assert len(got) == len(base)
        for a, b in zip(got, base):
            assert abs(a - b) < 2e-3, (kw, got, base)


@pytest.mark.dist
@pytest.mark.parametrize("layout", [dict(world_size=1), dict(world_size=2, mp=2), dict(world_size=2, pp=2, ga=2, micro=8),
                                    dict(world_size=2, zero=True)])
def test_resume_is_bit_identical(tmp_path: Path, layout):
    layout = dict(layout)
    ws = layout.pop("world_size")
    full = _losses(ws, iters=10, save_dir=str(tmp_path), save_interval=6, **layout)
    resumed = _losses(ws, iters=10, load_dir=str(tmp_path), **layout)
    assert len(resumed) == 4
    assert resumed == full[6:], (resumed, full[6:])


@pytest.mark.dist
def test_resume_into_other_layout(tmp_path: Path):
    full = _losses(2, mp=2, iters=10, save_dir=str(tmp_path), save_interval=6)
    for kw in (dict(world_size=1), dict(world_size=2, pp=2, ga=2, micro=8), dict(world_size=2, zero=True)):
        ws = kw.pop("world_size")
        resumed = _losses(ws, iters=10, load_dir=str(tmp_path), **kw)
        for a, b in zip(resumed, full[6:]):
            assert abs(a - b) < 2e-3, (kw, resumed, full[6:])


def _run_traced(rank, world_size, port, device, config, overlap):
    """Two training steps of the pipelined MLP; returns (losses, instruction trace of the second step)."""
    import os

    os.environ["SB200_PIPE_OVERLAP"] = "1" if overlap else "0"
    from scaling_b200.core.data import DataLoader
    from scaling_b200.core.runner import LaunchConfig
    from scaling_b200.models.mlp import (MLPConfig, MLPContext, SyntheticClassificationDataset, init_model,
                                         init_optimizer, loss_function, metrics_aggregation_fn)
    from scaling_b200.parallel import Topology

    lc = LaunchConfig(master_port=port, master_addr="127.0.0.1", world_size=world_size, global_rank=rank,
                      local_slot=rank, payload=copy.deepcopy(config))
    cfg = MLPConfig.from_dict(lc.overwrite_config_dict_with_launcher_args(dict(lc.payload)))
    topology = Topology(cfg.topology)
    context = MLPContext(config=cfg, topology=topology)
    context.initialize(master_addr="127.0.0.1", master_port=str(port), seed=cfg.trainer.seed)
    model = init_model(context)
    optimizer = init_optimizer(context, model)
    loader = None
    if topology.is_io_rank:
        dataset = SyntheticClassificationDataset(n_samples=cfg.data.n_samples, seed=cfg.trainer.seed)
        loader = DataLoader(seed=cfg.trainer.seed, consumed_samples=0, dataset=dataset, topology=topology)
    losses = []
    for step in range(3):
        model.instruction_trace = [] if step == 2 else None
        out = model.train_step(loader, optimizer, SyntheticClassificationDataset.sync_batch_to_model_parallel,
                               loss_function, metrics_aggregation_fn)
        losses.append(out.loss)
    return losses, model.instruction_trace


@pytest.mark.dist
def test_pipeline_receives_are_posted_ahead_of_the_compute_before_them():
    """With overlap on, a stage posts its next receive as soon as only compute lies between it and the receive's own
    instruction (never across one of its own sends, which the sender may be waiting for): the last stage gets the next
    activation while it runs forward and backward of the current micro batch, the first stage the next gradient while
    it runs a backward pass.  The losses are those of the run that posts every receive where the schedule names it."""
    config = _config(2, pp=2, ga=4, micro=4, iters=3)
    (loss_a, trace0), (_, trace1) = dist_launcher(_run_traced, 2, config=config, overlap=True)
    (loss_b, plain0), _ = dist_launcher(_run_traced, 2, config=config, overlap=False)
    assert loss_a == loss_b and loss_a[0] is not None
    assert not any(t.startswith("post ") for t in plain0)

    def pos(trace, entry):
        assert entry in trace, (entry, trace)
        return trace.index(entry)

    # last stage: activation of micro batch 1 is on its way while micro batch 0 is still being computed
    assert pos(trace1, "RecvActivation mb=0") < pos(trace1, "post RecvActivation mb=1") < pos(trace1, "ForwardPass mb=0")
    assert pos(trace1, "post RecvActivation mb=2") < pos(trace1, "ForwardPass mb=1")
    assert pos(trace1, "SendGrad mb=0") < pos(trace1, "post RecvActivation mb=2")  # not across the stage's own send
    # first stage, cool-down: the gradient of micro batch 3 is awaited while micro batch 2 runs backward
    assert pos(trace0, "RecvGrad mb=2") < pos(trace0, "post RecvGrad mb=3") < pos(trace0, "BackwardPass mb=2")
    assert pos(trace0, "SendActivation mb=1") < pos(trace0, "post RecvGrad mb=0")
    # every posted receive is consumed by its instruction, in order
    for trace, kind in ((trace1, "RecvActivation"), (trace0, "RecvGrad")):
        posted = [t.split("mb=")[1] for t in trace if t.startswith(f"post {kind}")]
        done = [t.split("mb=")[1] for t in trace if t.startswith(f"{kind} mb=")]
        assert posted == [m for m in done if m in posted] and len(posted) >= 3
