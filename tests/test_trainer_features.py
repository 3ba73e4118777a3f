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
    rows = profile["observations"]  # one record per timed instruction
    assert profile["pipe_parallel_size"] == 2 and profile["gradient_accumulation_steps"] == 2
    assert set(profile["fields"]) == set(rows[0])
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
    again = SimulationEngine(PipelineScheduleTrain, profile)  # the gathered record itself
    again.simulate()
    assert again.summarize()["total_time"] == engine.summarize()["total_time"]


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


def test_truncated_checkpoint_file_is_reported_not_loaded(tmp_path: Path):
    save = tmp_path / "ckpt"
    losses(1, save_dir=str(save), save_interval=2, iters=2)
    victim = sorted((save / "global_step2").glob("model_state_layer_1_*.pt"))[0]
    victim.write_bytes(victim.read_bytes()[:200])
    with pytest.raises(AssertionError, match="(?s)rank failures.*(Error|error)"):
        losses(1, load_dir=str(save), iters=3)


def test_a_killed_rank_takes_the_job_down_and_the_last_checkpoint_resumes_exactly(tmp_path: Path):
    """Failure on the host: one of two ranks is killed in the middle of training.  The launcher ends the other rank
    and reports the failure; a new job resumes from the last checkpoint and ends with the weights of a run that was
    never interrupted."""
    import os
    import signal
    import subprocess
    import sys
    import time

    import psutil
    import torch

    from scaling_b200.core.runner.launch_config import encode_base64
    from tests.utils import find_free_port

    root = Path(__file__).resolve().parent.parent
    reference = tmp_path / "reference"
    dist_launcher(run_training, 2, config=tiny_config(2, mp=2, iters=14, save_dir=str(reference), save_interval=14))

    crashed = tmp_path / "crashed"
    payload = tiny_config(2, mp=2, iters=1_000_000, save_dir=str(crashed), save_interval=10)
    pool = {"nodes": [{"name": "localhost", "slots": [0, 1]}], "world_size": 2}
    launcher = subprocess.Popen(
        [sys.executable, "-m", "scaling_b200.core.runner.launch", "--resource_pool", encode_base64(pool),
         "--master_port", str(find_free_port()), str(root / "scaling_b200" / "transformer" / "train.py"),
         "--payload", encode_base64(payload)], cwd=str(root), stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL,
        env=dict(os.environ, OMP_NUM_THREADS="1", MKL_NUM_THREADS="1"))  # one thread, as the in-process test ranks
    try:
        deadline = time.time() + 120
        while not (crashed / "global_step10" / "context_global_rank_1.pt").is_file() or not (crashed / "latest").is_file():
            assert launcher.poll() is None, "the job ended before its first checkpoint"
            assert time.time() < deadline, "no checkpoint within two minutes"
            time.sleep(0.2)
        children = psutil.Process(launcher.pid).children(recursive=False)
        assert len(children) == 2
        victim = children[1]
        victim.send_signal(signal.SIGKILL)  # this exact process: a rank that dies without a word
        rc = launcher.wait(timeout=60)
        assert rc != 0
        time.sleep(0.5)
        assert not any(c.is_running() and c.status() != psutil.STATUS_ZOMBIE for c in children)
    finally:
        if launcher.poll() is None:
            launcher.kill()
    (crashed / "latest").write_text("global_step10")  # later checkpoints may exist; resume from a known one
    resumed = tmp_path / "resumed"
    dist_launcher(run_training, 2, config=tiny_config(2, mp=2, iters=14, load_dir=str(crashed), save_dir=str(resumed),
                                                      save_interval=14))
    files = sorted(f.name for f in (reference / "global_step14").glob("model_state_layer_*.pt"))
    assert files
    for name in files:
        a = torch.load(reference / "global_step14" / name, map_location="cpu", weights_only=False)
        b = torch.load(resumed / "global_step14" / name, map_location="cpu", weights_only=False)
        assert a.keys() == b.keys()
        assert all(torch.equal(a[k], b[k]) for k in a), name


def test_checkpoint_layout_and_key_names(tmp_path: Path):
    """One model and one optimizer file per global layer index, module-path state keys, optimizer keys built from the
    parameter meta, a tied weight stored under each of its layer indices."""
    import torch

    save = tmp_path / "ckpt"
    losses(1, save_dir=str(save), save_interval=2, iters=2, arch={"weight_tying": True})
    step = save / "global_step2"
    names = sorted(f.name for f in step.iterdir())
    assert names == [
        "config.yml", "context_global_rank_0.pt",
        "model_state_layer_0_EmbeddingInput.pt", "model_state_layer_1_TransformerLayer.pt",
        "model_state_layer_2_TransformerLayer.pt", "model_state_layer_3_LayerNormWrapper.pt",
        "model_state_layer_4_TransformerLMHeadTied.pt",
        "optimizer_state_layer_0.pt", "optimizer_state_layer_1.pt", "optimizer_state_layer_2.pt",
        "optimizer_state_layer_3.pt", "optimizer_state_layer_4.pt", "parameter_meta_0_5.json"]
    block = torch.load(step / "model_state_layer_1_TransformerLayer.pt", weights_only=False)
    assert list(block) == ["input_layernorm.weight", "input_layernorm.bias", "self_attention.query_key_value.weight",
                           "self_attention.query_key_value.bias", "self_attention.dense.weight",
                           "self_attention.dense.bias", "post_attention_layernorm.weight",
                           "post_attention_layernorm.bias", "mlp.dense_in.weight", "mlp.dense_in.bias",
                           "mlp.dense_out.weight", "mlp.dense_out.bias"]
    first = torch.load(step / "optimizer_state_layer_0.pt", weights_only=False)
    last = torch.load(step / "optimizer_state_layer_4.pt", weights_only=False)
    assert set(first) == {"step_index", "loss_scaler", "parameters", "optimizer_param_groups"}
    key0 = "layer_index_0_parameter_name_embedding.weight_is_model_parallel_True_model_parallel_dimension_0"
    key4 = "layer_index_4_parameter_name_embedding.weight_is_model_parallel_True_model_parallel_dimension_0"
    assert list(first["parameters"]) == [key0] and list(last["parameters"]) == [key4]
    entry = first["parameters"][key0]
    assert set(entry) == {"parameter", "meta", "optimizer_state"}
    assert set(entry["optimizer_state"]) == {"step", "exp_avg", "exp_avg_sq"}
    assert entry["parameter"].dtype == torch.float32
    assert torch.equal(entry["parameter"], last["parameters"][key4]["parameter"])  # the tied copies are one weight
    meta = json.loads((step / "parameter_meta_0_5.json").read_text())
    assert any("embedding.weight" in str(k) or "embedding.weight" in str(v) for k, v in (meta.items() if isinstance(meta, dict) else enumerate(meta)))
    assert (save / "latest").read_text() == "global_step2"


def _count_worker(rank, world_size, port, device, config):
    import copy

    from scaling_b200.core.runner import LaunchConfig
    from scaling_b200.parallel import Topology
    from scaling_b200.transformer import TransformerConfig, TransformerContext, init_model

    lc = LaunchConfig(master_port=port, master_addr="127.0.0.1", world_size=world_size, global_rank=rank,
                      local_slot=rank, payload=copy.deepcopy(config))
    cfg = TransformerConfig.from_dict(lc.overwrite_config_dict_with_launcher_args(dict(lc.payload)))
    context = TransformerContext(config=cfg, topology=Topology(cfg.topology))
    context.initialize(master_addr="127.0.0.1", master_port=str(port), seed=1)
    return init_model(context).get_params_count()


@pytest.mark.parametrize("layout", [dict(world_size=1), dict(world_size=2, mp=2), dict(world_size=2, pp=2, ga=2, micro=2)])
def test_parameter_counts_do_not_depend_on_the_layout(layout):
    """Unique = every weight once (tied weights and copies replicated over the tensor-parallel ranks counted once):
    the same in every layout and on every rank.  Total = every stored copy."""
    h, v, layers = 64, 128, 2
    replicated = 2 * (2 * h) + h + h  # per block: two norms (weight, bias), attention-out bias, mlp-out bias
    block = (3 * h * h + 3 * h) + (h * h) + 2 * (4 * h * h) + 4 * h + replicated
    unique = v * h + layers * block + 2 * h + v * h
    kw = dict(layout)
    ws = kw.pop("world_size")
    mp = kw.get("mp", 1)
    copies = (mp - 1) * (layers * replicated + 2 * h)  # replicated parameters live on every tensor-parallel rank
    for tying, expected in ((False, (unique + copies, unique)), (True, (unique + copies, unique - v * h))):
        counts = dist_launcher(_count_worker, ws, config=tiny_config(ws, arch={"weight_tying": tying}, **kw))
        assert all(tuple(c) == expected for c in counts), (tying, counts, expected)


def _losses_with_evaluation(rank, world_size, port, device, config):
    from scaling_b200.core.runner import LaunchConfig
    from scaling_b200.transformer.train import main

    lc = LaunchConfig(master_port=port, master_addr="127.0.0.1", world_size=world_size, global_rank=rank,
                      local_slot=rank, payload=config)
    metrics = main(lc, return_metrics=True)
    return [{k: v for k, v in m.items() if k in ("training/loss", "evaluation/loss")} for m in metrics] if metrics else None


def test_evaluation_between_training_steps_agrees_across_layouts(tmp_path: Path):
    """Evaluation every second step on held-out data: the training and evaluation losses of a sequence-parallel and
    of a two-stage pipeline run equal those of one process."""
    init = str(tmp_path / "init")
    dist_launcher(run_training, 1, config=tiny_config(1, iters=1), save_initial=init)

    def config(ws, **kw):
        cfg = tiny_config(ws, iters=4, load_dir=init, **kw)
        cfg["trainer"].update(eval_interval=2, eval_iterations=2, load_optimizer_states=False, load_context=False)
        return cfg

    base = dist_launcher(_losses_with_evaluation, 1, config=config(1))[0]
    assert [sorted(m) for m in base] == [["training/loss"], ["evaluation/loss", "training/loss"]] * 2
    for kw in (dict(mp=2, sp=True), dict(pp=2, ga=2, micro=2)):
        got = dist_launcher(_losses_with_evaluation, 2, config=config(2, **kw))[0]
        for a, b in zip(got, base):
            assert a.keys() == b.keys()
            assert all(abs(a[k] - b[k]) < 2e-5 * max(1.0, abs(b[k])) for k in a), (kw, got, base)


def _run_with(load_dir, **trainer):
    cfg = tiny_config(1, iters=2, load_dir=str(load_dir))
    cfg["trainer"].update(trainer)
    return dist_launcher(run_training, 1, config=cfg)[0]


def test_older_layer_class_names_and_non_strict_loading(tmp_path: Path):
    """A checkpoint whose files carry the layer class names of the earlier code base loads like a current one; keys
    missing from or unknown to the model stop the load unless the config allows or ignores them."""
    import shutil

    import torch

    from scaling_b200.core.nn.parallel_module.partitioned_module import _is_legacy_checkpoint, legacy_checkpoint_mapping

    init = tmp_path / "init"
    base = losses(1, save_initial=str(init), iters=2)
    step = next(p for p in init.iterdir() if p.is_dir())

    old = tmp_path / "old"
    shutil.copytree(init, old)
    renamed = 0
    for f in sorted((old / step.name).glob("model_state_layer_*.pt")):
        for new_name, old_name in legacy_checkpoint_mapping.items():
            if f.name.endswith(f"_{new_name}.pt"):
                f.rename(f.with_name(f.name.replace(f"_{new_name}.pt", f"_{old_name}.pt")))
                renamed += 1
    assert renamed >= 3 and _is_legacy_checkpoint([old / step.name]) and not _is_legacy_checkpoint([step])
    assert _run_with(old) == base

    holes = tmp_path / "holes"
    shutil.copytree(init, holes)
    block = holes / step.name / "model_state_layer_1_TransformerLayer.pt"
    state = torch.load(block, weights_only=False)
    del state["mlp.dense_in.bias"]
    state["removed_module.weight"] = torch.zeros(3)
    torch.save(state, block)
    with pytest.raises(AssertionError, match="Unexpected keys in checkpoint"):
        _run_with(holes, load_optimizer_states=False)
    with pytest.raises(AssertionError, match="Missing keys in checkpoint"):
        _run_with(holes, load_optimizer_states=False, ignore_keys_in_checkpoint=["removed_module"])
    got = _run_with(holes, load_optimizer_states=False, ignore_keys_in_checkpoint=["removed_module"],
                    allowed_missing_keys_in_checkpoint=[r"dense_in\.bias"])
    assert len(got) == 2 and all(abs(a - b) < 0.05 for a, b in zip(got, base))
