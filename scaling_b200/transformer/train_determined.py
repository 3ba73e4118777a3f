"""Entry point of transformer training under Determined (src/scaling/transformer/train_determined.py:28-200).

The launcher provides rank information through the torch-distributed environment variables; hyper-parameters of the
trial are mapped onto config overrides (``hparams_to_overrides``), then the regular ``train.main`` runs with the
Determined context and profiler attached.
"""

from __future__ import annotations

import argparse
import os
from typing import Any, Optional, Union

from ..core.determined import determined_profiler_from_ctx, init, maybe_periodic_stacktraces
from ..core.runner import LaunchConfig
from .context.config import TransformerConfig
from .train import main as train_main

# hyper-parameter name -> (config section, key); values are copied as they are
_DIRECT = {
    "wandb_project": ("logger", "wandb_project"),
    "model_parallel_size": ("topology", "model_parallel_size"),
    "pipe_parallel_size": ("topology", "pipe_parallel_size"),
    "sequence_parallel": ("topology", "sequence_parallel"),
    "global_batch_size": ("topology", "global_batch_size"),
    "micro_batch_size": ("topology", "micro_batch_size"),
    "activation_checkpointing_type": ("topology", "activation_checkpointing_type"),
    "pipe_partition_method": ("topology", "pipe_partition_method"),
    "pipe_partition_overwrite": ("topology", "pipe_partition_overwrite"),
    "train_iterations": ("trainer", "train_iterations"),
    "sequence_length": ("transformer_architecture", "sequence_length"),
}


def from_launcher_args_determined() -> LaunchConfig:
    parser = argparse.ArgumentParser(description="process launch")
    parser.add_argument("--config", type=str, default=None, help="path to config file")
    parser.add_argument("remaining_args", nargs=argparse.REMAINDER)
    args = parser.parse_args()
    world_size = os.environ["WORLD_SIZE"]
    payload = None
    if args.config is not None:
        payload = TransformerConfig.from_yaml(
            args.config, overwrite_values={"topology": {"world_size": int(world_size)}}).as_dict()
    return LaunchConfig(master_addr=os.environ["MASTER_ADDR"], master_port=os.environ["MASTER_PORT"],
                        world_size=world_size, global_rank=os.environ["RANK"], local_slot=os.environ["LOCAL_RANK"],
                        payload=payload)


def hparams_to_overrides(hparams: Optional[dict], overwrite_config: Optional[dict] = None) -> dict:
    """Config overrides for a trial's hyper-parameters.  A ``layout`` entry (written when a single run is restarted)
    replaces the whole set.  Token budgets are converted to steps with the batch size and sequence length."""
    out: dict[str, Any] = dict(overwrite_config or {})
    if hparams and "layout" in hparams:
        hparams = hparams["layout"]
    if not hparams:
        return out
    for section in ("topology", "transformer_architecture", "logger", "trainer", "learning_rate_scheduler"):
        out.setdefault(section, {})
    if hparams.get("learning_rate"):
        out["learning_rate_scheduler"]["learning_rate"] = hparams["learning_rate"]
    for key, target in (("target_train_tokens", ("trainer", "train_iterations")),
                        ("warmup_tokens", ("learning_rate_scheduler", "learning_rate_warmup_steps"))):
        if hparams.get(key):
            assert "sequence_length" in hparams and "global_batch_size" in hparams
            out[target[0]][target[1]] = int(hparams[key] / (hparams["global_batch_size"] * hparams["sequence_length"]))
    for name, (section, key) in _DIRECT.items():
        if name in hparams:
            out[section][key] = hparams[name]
    if "kernel" in hparams:
        out["transformer_architecture"]["masked_softmax"] = {"kernel": hparams["kernel"]}
    return out


def main(determined_context: Any, profiler: Any, overwrite_config: Optional[dict] = None, return_metrics: bool = False,
         det_experiment_id: Optional[int] = None, det_trial_id: Optional[int] = None,
         info: Any = None) -> Optional[list[dict[str, Union[float, int]]]]:
    launch_config = from_launcher_args_determined()
    overrides = dict(overwrite_config or {})
    overrides.setdefault("runner", {})["use_determined"] = True
    overrides["determined_experiment_id"] = det_experiment_id
    overrides["determined_trial_id"] = det_trial_id
    overrides = hparams_to_overrides(info.trial.hparams if info is not None else None, overrides)
    return train_main(launch_config, overrides, return_metrics, determined_context, profiler)


if __name__ == "__main__":
    import determined as det

    info = det.get_cluster_info()
    assert info is not None
    config_determined = det.ExperimentConfig(info.trial._config)
    distributed = det.core.DistributedContext.from_torch_distributed()
    with maybe_periodic_stacktraces(config_determined.debug_enabled()):
        with init(distributed=distributed) as determined_context:
            with determined_profiler_from_ctx(determined_context, config_determined, info) as profiler:
                main(determined_context, profiler, det_experiment_id=info.trial.experiment_id,
                     det_trial_id=info.trial.trial_id, info=info)
