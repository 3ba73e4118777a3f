"""Training entry point of the transformer application.

``main(launch_config)``: config -> topology -> logger -> context (distributed init, seeds) -> model ->
optimizer -> datasets on IO ranks -> loss -> trainer -> training loop; run per rank by the launcher as
``python -m scaling_b200.transformer.train --payload <b64>`` (flow of
src/scaling/transformer/train.py:176-328).  The trainer additionally logs FLOP-model throughput, MFU
and tokens per second, and copies the tokenizer file into checkpoints.
"""

from __future__ import annotations

import os
import shutil
from pathlib import Path
from typing import Any, Callable, Optional

import torch

from ..core.logging import logger
from ..core.logging.logger_config import TensorboardRanksConfig
from ..core.nn.parallel_module import EvaluationStepOutput, TrainStepOutput
from ..core.runner import LaunchConfig
from ..core.trainer import BaseTrainer
from ..parallel.topology import Topology
from .context.config import DataConfig, TransformerConfig
from .context.context import TransformerContext
from .data.text_dataset import SyntheticTextDataset, TextDataset
from .model import TransformerParallelModule, init_model, init_optimizer, metrics_aggregation_fn
from .model.losses import create_loss_function
from .utils.get_tflops import (
    get_model_flop_utilization_palm,
    get_tflops_aleph_alpha,
    get_tflops_bloom,
    get_tflops_electra,
    get_tflops_megatron,
    get_tokens_per_second,
)


class TransformerTrainer(BaseTrainer[TransformerContext, TransformerParallelModule]):
    def save_checkpoint(self, save_dir: Optional[Path] = None) -> Path:
        save_dir = super().save_checkpoint(save_dir=save_dir)
        vocab_file = self.context.config.transformer_architecture.vocab_file
        if vocab_file is not None and save_dir is not None and self.context.topology.config.global_rank == 0:
            shutil.copy(vocab_file, Path(save_dir) / "vocab.json")
            # also beside the weights, where TransformerInferenceModule.from_checkpoint looks for it
            step_dir = Path(save_dir) / f"global_step{self.context.iterations}"
            if step_dir.is_dir():
                shutil.copy(vocab_file, step_dir / "vocab.json")
        return save_dir

    def _tflops_metrics(self, iter_time_s: float) -> dict[str, float]:
        a = self.context.config.transformer_architecture
        t = self.context.topology
        return {
            "runtime/tflops_megatron": get_tflops_megatron(self.parameters_total, iter_time_s, t, a),
            "runtime/tflops_megatron_layout_independent": get_tflops_megatron(self.parameters_unique, iter_time_s, t, a),
            "runtime/tflops_bloom": get_tflops_bloom(iter_time_s, t, a),
            "runtime/tflops_electra": get_tflops_electra(iter_time_s, t, a),
            "runtime/tflops_aleph_alpha": get_tflops_aleph_alpha(iter_time_s, t, a),
            "runtime/mfu_palm": get_model_flop_utilization_palm(iter_time_s, self.parameters_total, t, a),
            "runtime/tokens_per_second": get_tokens_per_second(iter_time_s, t, a),
        }

    def log_metrics(self, train_step_output: TrainStepOutput,
                    eval_step_output: Optional[EvaluationStepOutput] = None) -> dict[str, Any]:
        t = train_step_output
        metrics: dict[str, Any] = {"training/loss": t.loss, "runtime/step_duration": t.step_duration}
        metrics.update(t.debug_dict or {})
        metrics.update(t.metrics or {})
        for key, value in (("training/global_grad_norm", t.global_grad_norm),
                           ("training/global_grad_norm_clipped", t.global_grad_norm_clipped),
                           ("training/overflow", None if t.overflow is None else int(t.overflow)),
                           ("training/no_overflow_steps", t.no_overflow_steps),
                           ("training/current_loss_scale", t.current_loss_scale)):
            if value is not None:
                metrics[key] = value
        for name, lr in (t.learning_rates or {}).items():
            metrics[f"training/learning_rate_{name}"] = lr
        metrics.update(self._tflops_metrics(t.step_duration))
        if eval_step_output is not None:
            for k, v in (eval_step_output.metrics or {}).items():
                metrics[f"evaluation/{k}"] = v
            metrics["evaluation/loss"] = eval_step_output.loss
            metrics["evaluation/step_duration"] = eval_step_output.step_duration
        logger.log_metrics(metrics, step=self.context.iterations)
        return metrics


def _enable_deterministic_torch() -> None:
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    torch.use_deterministic_algorithms(True)


def _init_transformer_config(launch_config: LaunchConfig, overwrite_config: Optional[dict[str, Any]]) -> TransformerConfig:
    config_dict = dict(launch_config.payload or overwrite_config or {})
    config_dict = launch_config.overwrite_config_dict_with_launcher_args(config_dict)
    return TransformerConfig.from_dict(config_dict, overwrite_values=overwrite_config if launch_config.payload else None)


def _init_logger(config: TransformerConfig, determined_context: Any, topology: Topology) -> None:
    ranks = config.logger.tensorboard_ranks
    if isinstance(ranks, TensorboardRanksConfig):
        ranks = topology.get_global_rank_group(data_parallel_rank=ranks.data_parallel_rank,
                                               model_parallel_rank=ranks.model_parallel_rank,
                                               pipe_parallel_rank=ranks.pipe_parallel_rank)
    name = f"RANK {topology.config.global_rank}"
    if config.runner.use_determined and determined_context is not None:
        logger.configure_determined(config=config.logger, name=name, global_rank=topology.config.global_rank,
                                    determined_context=determined_context, tensorboard_ranks=ranks)
    else:
        logger.configure(config=config.logger, name=name, global_rank=topology.config.global_rank,
                         tensorboard_ranks=ranks)
    logger.log_config(config=config)


def _get_sync_batch(data_config: DataConfig) -> Callable:
    if data_config.finetuning_dataset:
        from .data.finetuning_text_dataset import FinetuningTextDataset

        return FinetuningTextDataset.sync_batch_to_model_parallel
    if data_config.finetuning_chat_dataset:
        from .data.finetuning_chat_dataset import FinetuningChatDataset

        return FinetuningChatDataset.sync_batch_to_model_parallel
    if data_config.embedding_dataset:
        from .data.embedding_dataset import EmbeddingDataset

        return EmbeddingDataset.sync_batch_to_model_parallel
    return TextDataset.sync_batch_to_model_parallel


def _read_datasets(config: TransformerConfig):
    d, a = config.data, config.transformer_architecture
    seed = config.trainer.seed
    if not d.data_prefixes:
        n = d.synthetic_samples or 8 * config.topology.global_batch_size
        train = SyntheticTextDataset(n_samples=n, sequence_length=a.sequence_length, vocab_size=a.vocab_size, seed=seed,
                                     low=1, reset_attention_mask=a.reset_attention_mask,
                                     reset_position_ids=a.reset_position_ids)
        validation = None
        if config.trainer.eval_interval is not None:  # held-out synthetic samples: evaluation works without data files
            validation = SyntheticTextDataset(n_samples=max(64, n // 8), sequence_length=a.sequence_length,
                                              vocab_size=a.vocab_size, seed=seed + 1, low=1,
                                              reset_attention_mask=a.reset_attention_mask,
                                              reset_position_ids=a.reset_position_ids)
        return train, validation
    from .dataset_loader import load_blended_datasets

    return load_blended_datasets(config)


def main(launch_config: LaunchConfig, overwrite_config: Optional[dict[str, Any]] = None, return_metrics: bool = False,
         determined_context: Any = None, determined_profiler: Any = None) -> Optional[list[dict[str, Any]]]:
    config = _init_transformer_config(launch_config, overwrite_config)
    topology = Topology(config=config.topology)
    _init_logger(config, determined_context, topology)
    if config.training.use_deterministic_torch_algorithms:
        _enable_deterministic_torch()
    context = TransformerContext(config=config, topology=topology)
    if determined_context is not None:
        context.initialize_with_determined(
            master_addr=launch_config.master_addr, master_port=str(launch_config.master_port),
            determined_context=determined_context, determined_profiler=determined_profiler, seed=config.trainer.seed,
        )
    else:
        context.initialize(master_addr=launch_config.master_addr, master_port=str(launch_config.master_port),
                           seed=config.trainer.seed)
    model = init_model(context=context)
    optimizer = init_optimizer(context=context, model=model)
    dataset = validation = None
    if topology.is_io_rank:
        dataset, validation = _read_datasets(config)
    trainer = TransformerTrainer(
        config=config.trainer, context=context, parallel_module=model, optimizer=optimizer, dataset=dataset,
        sync_batch_to_model_parallel=_get_sync_batch(config.data),
        loss_function=create_loss_function(context, config.training.loss_function_config),
        metrics_aggregation_fn=metrics_aggregation_fn, dataset_evaluation=validation,
    )
    return trainer.run_training(return_metrics=return_metrics)


if __name__ == "__main__":
    main(LaunchConfig.from_launcher_args())
