"""The per-node launcher with real local processes, the example configs, and the MLP application started the way
the runner starts it (one process per slot, config in the base64 payload, gloo ranks on CPU)."""

import json
import sys
import textwrap
from pathlib import Path

import pytest
import yaml

from scaling_b200.core.runner.launch import local_assignment
from scaling_b200.core.runner.launch import main as launch_main
from scaling_b200.core.runner.launch_config import decode_base64, encode_base64
from tests.utils import find_free_port

ROOT = Path(__file__).resolve().parent.parent


def _pool(*slots_per_node):
    nodes = [{"name": f"node{i}", "slots": list(range(n))} for i, n in enumerate(slots_per_node)]
    return {"nodes": nodes, "world_size": sum(slots_per_node)}


def test_payload_round_trip_and_rank_assignment():
    payload = {"a": [1, 2, {"b": "c"}], "x": None}
    assert decode_base64(encode_base64(payload)) == payload
    slots, ranks, world = local_assignment(_pool(2, 3), node_rank=1)
    assert (slots, ranks, world) == ([0, 1, 2], [2, 3, 4], 5)


def test_launcher_starts_one_process_per_slot_with_its_launch_config(tmp_path: Path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import json, sys
        sys.path.insert(0, {str(ROOT)!r})
        from scaling_b200.core.runner import LaunchConfig
        lc = LaunchConfig.from_launcher_args()
        open({str(tmp_path)!r} + f"/rank_{{lc.global_rank}}.json", "w").write(lc.as_str())
    """))
    rc = launch_main(["--resource_pool", encode_base64(_pool(3)), "--node_rank", "0", "--master_port", "29999",
                      str(script), "--payload", encode_base64({"hello": "world"})])
    assert rc == 0
    seen = [json.loads((tmp_path / f"rank_{r}.json").read_text()) for r in range(3)]
    assert [s["global_rank"] for s in seen] == [0, 1, 2] and [s["local_slot"] for s in seen] == [0, 1, 2]
    assert all(s["world_size"] == 3 and s["master_port"] == 29999 and s["payload"] == {"hello": "world"} for s in seen)


def test_launcher_stops_the_job_when_a_rank_fails(tmp_path: Path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent("""
        import os, sys, time
        if os.environ["RANK"] == "1":
            sys.exit(3)
        time.sleep(60)
    """))
    rc = launch_main(["--resource_pool", encode_base64(_pool(2)), str(script)])
    assert rc == 3  # the sleeping rank was terminated instead of being waited for


@pytest.mark.parametrize("name,cls_path", [
    ("mlp_example", "scaling_b200.models.mlp.MLPConfig"),
    ("transformer_example", "scaling_b200.transformer.TransformerConfig"),
])
def test_example_configs_parse(name, cls_path):
    import importlib

    module, cls = cls_path.rsplit(".", 1)
    config_cls = getattr(importlib.import_module(module), cls)
    config = config_cls.from_yaml(ROOT / "examples" / name / "config.yml")
    assert config.runner.script is not None and (ROOT / config.runner.script).is_file()
    again = config_cls.from_dict(config.as_dict())
    for field in type(config).model_fields:
        if field != "logger":  # the logger config stamps the wandb group with the time of its creation
            assert getattr(again, field) == getattr(config, field), field


@pytest.mark.dist
def test_mlp_example_trains_when_started_by_the_launcher(tmp_path: Path):
    payload = yaml.safe_load((ROOT / "examples" / "mlp_example" / "config.yml").read_text())
    payload["trainer"].update(train_iterations=3, save_dir=str(tmp_path / "ckpt"), save_interval=3)
    payload["topology"].update(device="cpu", backend="gloo")
    payload.setdefault("logger", {})["log_dir"] = str(tmp_path / "logs")
    rc = launch_main(["--resource_pool", encode_base64(_pool(2)), "--master_port", str(find_free_port()),
                      str(ROOT / payload["runner"]["script"]), "--payload", encode_base64(payload)])
    assert rc == 0
    step_dir = tmp_path / "ckpt" / "global_step3"
    assert (tmp_path / "ckpt" / "latest").read_text().strip() == "global_step3"
    assert any(step_dir.glob("model_state_layer_*.pt")) and any(step_dir.glob("optimizer_state_layer_*.pt"))
    assert (step_dir / "context_global_rank_0.pt").is_file() and (step_dir / "context_global_rank_1.pt").is_file()


@pytest.mark.dist
def test_transformer_training_script_under_the_launcher(tmp_path: Path):
    """The transformer entry point as the runner starts it: pipeline of two stages, evaluation and a checkpoint."""
    from tests.test_transformer_training import tiny_config

    import numpy as np

    from scaling_b200.core.data import MemoryMapDatasetBuilder

    rng = np.random.default_rng(0)
    for name, docs in (("train", 80), ("valid", 30)):  # token files as the tokeniser script leaves them (0 = end of document)
        with MemoryMapDatasetBuilder(prefix_path=tmp_path / name) as b:
            for _ in range(docs):
                b.add(np_array=np.concatenate([rng.integers(1, 128, size=rng.integers(5, 60)), [0]]).astype(np.int32))
    payload = tiny_config(2, pp=2, ga=2, micro=2, iters=2, save_dir=str(tmp_path / "ckpt"), save_interval=2)
    payload["trainer"].update(eval_interval=2, eval_iterations=1)
    payload["data"] = {"data_prefixes": [str(tmp_path / "train")], "validation_data_prefixes": [str(tmp_path / "valid")]}
    payload["logger"] = {"log_dir": str(tmp_path / "logs")}
    rc = launch_main(["--resource_pool", encode_base64(_pool(2)), "--master_port", str(find_free_port()),
                      str(ROOT / "scaling_b200" / "transformer" / "train.py"), "--payload", encode_base64(payload)])
    assert rc == 0
    step_dir = tmp_path / "ckpt" / "global_step2"
    names = sorted(f.name for f in step_dir.glob("model_state_layer_*.pt"))
    # embedding, two blocks, final norm, head: one file per layer whatever stage holds it
    assert [n.split("_")[3] for n in names] == ["0", "1", "2", "3", "4"], names
    assert (step_dir / "config.yml").is_file()


def test_mlp_example_modules_are_importable_under_the_example_layout():
    import yaml

    from examples.mlp_example import context, data, model, train
    from examples.mlp_example.config import MLPConfig

    cfg = MLPConfig.from_dict(yaml.safe_load((Path(__file__).parents[1] / "examples/mlp_example/config.yml").read_text()))
    assert cfg.architecture.hidden_dim > 0
    assert callable(train.main) and hasattr(model, "get_layer_specs") and hasattr(data, "MNISTDataset")
    assert context.MLPContext.__name__ == "MLPContext"
