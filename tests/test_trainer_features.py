"""Trainer-level behaviour on CPU ranks: fp16 with dynamic loss scaling, the step profiler, checkpoint housekeeping,
per-rank log files."""

import json
from pathlib import Path

import pytest

from tests.test_transformer_training import losses, run_training, tiny_config
from tests.utils import dist_launcher

pytestmark = pytest.mark.dist


def test_fp16_training_with_dynamic_loss_scaling_resumes_exactly(tmp_path: Path):
    """Half precision with the dynamic loss scaler: the first steps overflow at a huge initial scale and are skipped
    (the scale halves), training then proceeds; a resumed run repeats the original losses bit for bit."""
    arch = {"precision": "float16"}
    save = str(tmp_path / "ckpt")

    def config(**kw):
        cfg = tiny_config(2, mp=2, arch=arch, **kw)
        cfg["optimizer"]["loss_scaler"] = {"enable": True, "initial_scale": 2.0 ** 24, "window": 2, "hysteresis": 1,
                                           "factor": 2.0, "min_scale": 1.0}
        return cfg

    full = dist_launcher(run_training, 2, config=config(iters=8))[0]
    first = dist_launcher(run_training, 2, config=config(iters=4, save_dir=save, save_interval=4))[0]
    resumed = dist_launcher(run_training, 2, config=config(iters=8, load_dir=save))[0]
    assert all(l == l for l in full)
    assert first == full[:4] and resumed == full[4:], (first, resumed, full)


def _profiled(rank, world_size, port, device, config):
    out = run_training(rank, world_size, port, device, config)
    return out


def test_profiler_writes_per_instruction_timings_under_pipeline_parallelism(tmp_path: Path):
    cfg = tiny_config(2, pp=2, ga=2, micro=2, iters=4)
    cfg["profiler"] = {"profile_steps": 2, "profile_start_at_step": 1, "profiler_output": str(tmp_path / "profile.json")}
    dist_launcher(_profiled, 2, config=cfg)
    profile = json.loads((tmp_path / "profile.json").read_text())
    fields = profile["fields"]
    rows = [dict(zip(fields, r)) for r in profile["observations"]]
    names = {r["timer_name"] for r in rows}
    assert {"ForwardPass", "BackwardPass", "SendActivation", "RecvActivation"} <= names, names
    assert {r["pipe_parallel_rank"] for r in rows} == {0, 1}  # gathered from both stages on rank 0
    assert all(r["duration"] >= 0 for r in rows)
    # the recorded durations drive the schedule simulator (timeline of the measured run)
    from scaling_b200.core.nn.pipeline_schedule import PipelineScheduleTrain
    from scaling_b200.core.nn.pipeline_schedule.simulator import SimulationEngine

    engine = SimulationEngine.from_profile(PipelineScheduleTrain, tmp_path / "profile.json")
    engine.simulate()
    assert engine.summarize()["total_time"] > 0


def test_past_optimizer_states_are_deleted_and_latest_points_to_the_last_checkpoint(tmp_path: Path):
    save = tmp_path / "ckpt"
    cfg = tiny_config(1, iters=4, save_dir=str(save), save_interval=2)
    cfg["trainer"]["delete_past_optimizer_states"] = True
    dist_launcher(run_training, 1, config=cfg)
    assert (save / "latest").read_text().strip() == "global_step4"
    assert not list((save / "global_step2").glob("optimizer_state_*.pt"))
    assert list((save / "global_step2").glob("model_state_layer_*.pt"))  # the weights of older checkpoints stay
    assert list((save / "global_step4").glob("optimizer_state_*.pt"))
    # the kept checkpoint resumes
    assert len(losses(1, load_dir=str(save), iters=6)) == 2


def _main_entry(rank, world_size, port, device, config):
    from scaling_b200.core.runner import LaunchConfig
    from scaling_b200.transformer.train import main

    lc = LaunchConfig(master_port=port, master_addr="127.0.0.1", world_size=world_size, global_rank=rank,
                      local_slot=rank, payload=config)
    metrics = main(lc, return_metrics=True)
    return [m["training/loss"] for m in metrics] if metrics else None


def test_every_rank_writes_its_own_log_file(tmp_path: Path):
    cfg = tiny_config(2, mp=2, iters=1)
    cfg["logger"] = {"log_dir": str(tmp_path / "logs")}
    dist_launcher(_main_entry, 2, config=cfg)
    files = sorted(p.name for p in (tmp_path / "logs").rglob("*") if p.is_file())
    assert len(files) >= 2, files
