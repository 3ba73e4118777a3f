"""Training loop around a ParallelModule and an Optimizer.

Responsibilities (reference: src/scaling/core/trainer/trainer.py:33-330): count parameters, load a
checkpoint (``load_dir/latest`` names the ``global_step{N}`` directory; a flat directory of ``.pt``
files also works), optionally merge LoRA weights, create data loaders on IO ranks resuming from the
consumed-sample counter, then loop: train step -> checkpoint every ``save_interval`` -> evaluation
every ``eval_interval`` -> metrics on rank 0.  Checkpoints are written to
``save_dir/global_step{N}`` and ``save_dir/latest`` is updated by rank 0.
"""

from __future__ import annotations

from contextlib import nullcontext
from pathlib import Path
from typing import Any, Callable, Dict, Generic, List, Optional, TypeVar, Union

import torch
import torch.distributed as dist

from ..context import BaseContextGeneric
from ..data import BaseDataset, DataLoader
from ..logging import logger
from ..nn.parallel_module import EvaluationStepOutput, ParallelModule, TrainStepOutput
from ..optimizer import BaseOptimizer
from .trainer_config import TrainerConfig

ParallelModuleGeneric = TypeVar("ParallelModuleGeneric", bound=ParallelModule)


class BaseTrainer(Generic[BaseContextGeneric, ParallelModuleGeneric]):
    def __init__(self, config: TrainerConfig, context: BaseContextGeneric, parallel_module: ParallelModuleGeneric,
                 optimizer: BaseOptimizer, dataset: Optional[BaseDataset], sync_batch_to_model_parallel: Callable,
                 loss_function: Callable, metrics_aggregation_fn: Optional[Callable] = None,
                 dataset_evaluation: Optional[BaseDataset] = None):
        self.config = config
        self.context = context
        self.parallel_module = parallel_module
        self.optimizer = optimizer
        self.dataset = dataset
        self.dataset_evaluation = dataset_evaluation
        self.sync_batch_to_model_parallel = sync_batch_to_model_parallel
        self.loss_function = loss_function
        self.metrics_aggregation_fn = metrics_aggregation_fn
        self.parameters_total, self.parameters_unique = parallel_module.get_params_count()
        logger.log_config_dict({"parameters_total": self.parameters_total, "parameters_unique": self.parameters_unique})

        loaded = self.load_checkpoint(
            load_dir=config.load_dir, load_optimizer_states=config.load_optimizer_states,
            load_context=config.load_context,
            allowed_missing_keys_in_checkpoint=config.allowed_missing_keys_in_checkpoint,
            allowed_unexpected_keys_in_checkpoint=config.allowed_unexpected_keys_in_checkpoint,
            ignore_keys_in_checkpoint=config.ignore_keys_in_checkpoint,
        )
        if config.assert_checkpoint_loaded and config.load_dir is not None:
            assert loaded, (
                "checkpoint could not be loaded. if this is intended you may change the parameter "
                "'assert_checkpoint_loaded' in the TrainerConfig to False."
            )
        if config.merge_lora_after_loading_checkpoint:
            for module in parallel_module.modules():
                if hasattr(module, "merge_lora_weights") and getattr(module, "lora_config", None):
                    module.merge_lora_weights()
            optimizer.refresh_optimizer_after_model_change()
            logger.info("Merged LoRa weights")

        # data loaders are created after the checkpoint load so that they resume at the right sample
        self.dataloader: Optional[DataLoader] = None
        self.dataloader_evaluation: Optional[DataLoader] = None
        if context.topology.is_io_rank:
            assert dataset is not None, "io ranks need a dataset"
            self.dataloader = self._make_loader(dataset, context.consumed_samples)
            if dataset_evaluation is not None:
                self.dataloader_evaluation = self._make_loader(dataset_evaluation, context.consumed_samples_evaluation)

        if config.delete_past_optimizer_states and config.save_dir is not None:
            logger.warning(
                "delete_past_optimizer_states is set: optimizer states of all checkpoints but the latest are deleted "
                "every time a checkpoint is saved; set the flag to false to keep them"
            )
        self.tensor_statistics_recorder = None
        if config.tensor_statistics_recorder_config is not None:
            from ..logging.tensor_statistics_recorder import TensorStatisticsRecorder, TensorStatisticsRecorderConfig

            rc = config.tensor_statistics_recorder_config
            if isinstance(rc, dict):
                rc = TensorStatisticsRecorderConfig.from_dict(rc)
            self.tensor_statistics_recorder = TensorStatisticsRecorder(config=rc, context=context, model=parallel_module)

    def _make_loader(self, dataset: BaseDataset, consumed: int) -> DataLoader:
        c = self.config
        return DataLoader(seed=c.seed, consumed_samples=consumed, dataset=dataset, topology=self.context.topology,
                          num_workers=c.dataloader_num_workers, pin_memory=c.dataloader_pin_memory,
                          prefetch_factor=c.dataloader_prefetch_factor)

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, save_dir: Optional[Path] = None) -> Path:
        save_dir = Path(save_dir or self.config.save_dir)  # type: ignore[arg-type]
        iteration_dir = save_dir / f"global_step{self.context.iterations}"
        iteration_dir.mkdir(exist_ok=True, parents=True)
        self.parallel_module.save_checkpoint(iteration_dir,
                                             separate_file_for_parameters=self.config.separate_file_for_parameters)
        self.optimizer.save_checkpoint(iteration_dir)
        self.context.save_checkpoint(iteration_dir)
        topo = self.context.topology
        if topo.is_distributed_initialized and topo.world_size > 1:
            dist.barrier()
        if topo.config.global_rank == 0:
            (save_dir / "latest").write_text(f"global_step{self.context.iterations}", encoding="UTF-8")
            if self.config.delete_past_optimizer_states:
                self._delete_past_optimizer_states(save_dir, keep=iteration_dir)
        logger.info(f"saved checkpoint: {iteration_dir}")
        return save_dir

    @staticmethod
    def _delete_past_optimizer_states(save_dir: Path, keep: Path) -> None:
        for d in save_dir.glob("global_step*"):
            if d.is_dir() and d != keep:
                for f in d.glob("optimizer_state_*.pt"):
                    f.unlink(missing_ok=True)

    def load_checkpoint(self, load_dir: Optional[Path] = None, load_optimizer_states: bool = True,
                        load_context: bool = True, allowed_missing_keys_in_checkpoint: Optional[List[str]] = None,
                        allowed_unexpected_keys_in_checkpoint: Optional[List[str]] = None,
                        ignore_keys_in_checkpoint: Optional[List[str]] = None) -> bool:
        if load_dir is None:
            return False
        load_dir = Path(load_dir)
        if (load_dir / "latest").is_file():
            iteration_dir = load_dir / (load_dir / "latest").read_text(encoding="UTF-8").strip()
        elif any(load_dir.glob("*.pt")):
            logger.info(f"no latest file found, using load dir directly instead: {load_dir}")
            iteration_dir = load_dir
        else:
            logger.error(f"no files found in load dir: {load_dir}")
            return False
        if not iteration_dir.is_dir():
            logger.error(f"iteration_dir does not exist: {iteration_dir}")
            return False
        self.parallel_module.load_checkpoint(
            iteration_dir, allowed_missing_keys_in_checkpoint=allowed_missing_keys_in_checkpoint,
            allowed_unexpected_keys_in_checkpoint=allowed_unexpected_keys_in_checkpoint,
            ignore_keys_in_checkpoint=ignore_keys_in_checkpoint,
        )
        if load_optimizer_states:
            # a step captured earlier holds the addresses of the optimizer's per-step scalars, which a load may replace
            release = getattr(self.parallel_module, "release_cuda_graph", None)
            if release is not None:
                release()
            self.optimizer.load_checkpoint(iteration_dir)
        else:
            self.optimizer.refresh_optimizer_after_model_change()
        if load_context:
            self.context.load_checkpoint(iteration_dir)
        logger.info(f"loaded checkpoint: {iteration_dir}")
        return True

    # ------------------------------------------------------------------ extension points of the loop
    def _before_train_step(self) -> None:
        """Called at the top of every iteration of ``run_training``."""

    def _after_train_step(self) -> None:
        """Called right after the training step, before checkpointing and evaluation."""

    def _saves_without_save_dir(self) -> bool:
        """True when checkpoints have a destination other than ``config.save_dir``."""
        return False

    # ------------------------------------------------------------------ steps
    def train_step(self) -> TrainStepOutput:
        out = self.parallel_module.train_step(
            dataloader=self.dataloader, optimizer=self.optimizer,
            sync_batch_to_model_parallel=self.sync_batch_to_model_parallel, loss_function=self.loss_function,
            metrics_aggregation_fn=self.metrics_aggregation_fn,
        )
        self.context.step()
        return out

    def eval_step(self) -> EvaluationStepOutput:
        if self.context.topology.is_io_rank:
            assert self.dataloader_evaluation is not None, (
                "needs an evaluation dataloader on io ranks if evaluation is to be performed. "
                "Remember to give the trainer a dataset_evaluation"
            )
        return self.parallel_module.evaluation_step(
            dataloader=self.dataloader_evaluation, sync_batch_to_model_parallel=self.sync_batch_to_model_parallel,
            loss_function=self.loss_function, metrics_aggregation_fn=self.metrics_aggregation_fn,
        )

    def log_metrics(self, train_step_output: TrainStepOutput,
                    eval_step_output: Optional[EvaluationStepOutput]) -> Dict[str, Any]:
        t = train_step_output
        metrics: Dict[str, Any] = {f"training/{k}": v for k, v in (t.metrics or {}).items()}
        assert "training/loss" not in metrics
        metrics["training/loss"] = t.loss
        metrics["training/step_duration"] = t.step_duration
        optional = {
            "training/global_grad_norm": t.global_grad_norm,
            "training/global_grad_norm_clipped": t.global_grad_norm_clipped,
            "training/overflow": None if t.overflow is None else int(t.overflow),
            "training/no_overflow_steps": t.no_overflow_steps,
            "training/current_loss_scale": t.current_loss_scale,
        }
        metrics.update({k: v for k, v in optional.items() if v is not None})
        for name, lr in (t.learning_rates or {}).items():
            metrics[f"training/learning_rate_{name}"] = lr
        if eval_step_output is not None:
            for k, v in (eval_step_output.metrics or {}).items():
                metrics[f"evaluation/{k}"] = v
            metrics["evaluation/loss"] = eval_step_output.loss
            metrics["evaluation/step_duration"] = eval_step_output.step_duration
        logger.log_metrics(metrics, step=self.context.iterations)
        return metrics

    def run_training(self, return_metrics: bool = False) -> Optional[List[Dict[str, Union[float, int]]]]:
        collected: List[Dict[str, Any]] = []
        c = self.config
        while self.context.iterations < (c.train_iterations or 0):
            recorder = nullcontext()
            rec = self.tensor_statistics_recorder
            if rec is not None and self.context.iterations % rec.config.interval == 0:
                recorder = rec.trace()
            self._before_train_step()
            with recorder:
                train_out = self.train_step()
            self._after_train_step()
            if (c.save_interval is not None and (c.save_dir is not None or self._saves_without_save_dir())
                    and self.context.iterations % c.save_interval == 0):
                self.save_checkpoint()
            eval_out = None
            if c.eval_interval is not None and self.context.iterations % c.eval_interval == 0:
                eval_out = self.eval_step()
            if self.context.topology.config.global_rank == 0:
                metrics = self.log_metrics(train_out, eval_out)
                if return_metrics:
                    collected.append(metrics)
        # a captured training step holds communicators and static buffers; training is over, let them go so that
        # process groups can be destroyed
        release = getattr(self.parallel_module, "release_cuda_graph", None)
        if release is not None:
            release()
        return collected if return_metrics else None


class DeterminedBaseTrainer(BaseTrainer[BaseContextGeneric, ParallelModuleGeneric]):
    """Trainer for runs managed by Determined (src/scaling/core/trainer/trainer.py:336-560): checkpoints go through the
    experiment's storage manager and are reported to the master, a paused / restarted trial resumes from the
    master's latest checkpoint, and a preemption request is answered with a checkpoint and a clean exit.  Without a
    Determined context on ``self.context`` it behaves exactly like ``BaseTrainer``."""

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        if self._determined() and self.context.topology.config.global_rank == 0:
            self.delete_preempted_checkpoints_determined()

    def _determined(self) -> bool:
        return bool(getattr(self.context, "_use_determined", False))

    def _saves_without_save_dir(self) -> bool:
        return self._determined()

    def _before_train_step(self) -> None:
        profiler = getattr(self.context, "determined_profiler", None)
        if self._determined() and profiler is not None:
            profiler.update_batch_idx(self.context.iterations)

    def _after_train_step(self) -> None:
        if not self._determined():
            return
        ctx = self.context.determined_context
        assert ctx is not None
        if ctx.preempt.should_preempt():
            self.determined_save_checkpoint()
            logger.info("exiting program after preemption.")
            raise SystemExit(0)

    def save_checkpoint(self, save_dir: Optional[Path] = None) -> Path:
        if self._determined():
            return self.determined_save_checkpoint()
        return super().save_checkpoint(save_dir=save_dir)

    def determined_save_checkpoint(self) -> Path:
        """Rank 0 opens a storage path and broadcasts it; every rank writes its files there; files of nodes without
        a shared file system are gathered before the checkpoint is reported."""
        import uuid

        from determined.common import storage

        ctx = self.context.determined_context
        assert ctx is not None, "tried to save Determined checkpoint but no determined context is given"
        manager = ctx.checkpoint._storage_manager
        shared = isinstance(manager, storage.SharedFSStorageManager)
        if self.context.topology.config.global_rank == 0:
            storage_id = str(uuid.uuid4())
            with manager.store_path(storage_id) as path:
                ctx.distributed.broadcast((storage_id, path))
                BaseTrainer.save_checkpoint(self, save_dir=path)
                resources = storage.StorageManager._list_directory(path)
                gathered = [resources] if shared else ctx.distributed.gather(resources)
            merged = {k: v for d in gathered for k, v in d.items()}
            ctx.checkpoint._report_checkpoint(storage_id, merged, {"steps_completed": self.context.iterations})
            if self.config.delete_past_optimizer_states:
                self.delete_previous_optimizer_states_determined(storage_id)
        else:
            storage_id, path = ctx.distributed.broadcast(None)
            BaseTrainer.save_checkpoint(self, save_dir=path)
            if not shared:
                local = storage.StorageManager._list_directory(path) if ctx.distributed.local_rank == 0 else {}
                ctx.distributed.gather(local)
            if ctx.distributed.local_rank == 0:
                manager.post_store_path(str(path), storage_id)
        return Path(path)

    def load_checkpoint(self, load_dir: Optional[Path] = None, load_optimizer_states: bool = True,  # type: ignore[override]
                        load_context: bool = True, **kwargs: Any) -> bool:
        resumed = False
        if self._determined():
            import determined as det

            info = det.get_cluster_info()
            if info is not None and info.latest_checkpoint is not None:
                resumed = True
                with self.context.determined_context.checkpoint.restore_path(info.latest_checkpoint) as path:
                    logger.info(f"Updating load checkpoint directory from {self.config.load_dir} to {path} "
                                "according to determined setting")
                    return super().load_checkpoint(load_dir=Path(path), load_optimizer_states=True, load_context=True,
                                                   **kwargs)
        return super().load_checkpoint(load_dir=load_dir, load_optimizer_states=load_optimizer_states or resumed,
                                       load_context=load_context or resumed, **kwargs)

    def delete_preempted_checkpoints_determined(self) -> None:
        """Remove checkpoints that earlier preemptions of this trial left behind (all but the latest)."""
        import os

        if os.environ.get("DETERMINED_TEST", None) == "True":
            return
        try:
            import determined as det
            from determined.experimental import client

            info = det.get_cluster_info()
            if info is None:
                return
            trial = client.get_trial(info.trial.trial_id)
            checkpoints = trial.list_checkpoints() if hasattr(trial, "list_checkpoints") else trial.get_checkpoints()
            for ckpt in checkpoints:
                if ckpt.uuid != info.latest_checkpoint:
                    ckpt.delete()
        except Exception as e:  # noqa: BLE001 - clean-up must never stop a run
            logger.warning(f"could not delete preempted checkpoints: {e}")

    def delete_previous_optimizer_states_determined(self, keep_storage_id: str) -> None:
        """Drop optimizer-state files from this trial's older checkpoints (keeps the model weights)."""
        try:
            import determined as det
            from determined.experimental import client

            info = det.get_cluster_info()
            if info is None:
                return
            trial = client.get_trial(info.trial.trial_id)
            checkpoints = trial.list_checkpoints() if hasattr(trial, "list_checkpoints") else trial.get_checkpoints()
            for ckpt in checkpoints:
                if ckpt.uuid != keep_storage_id:
                    ckpt.remove_files(["**/optimizer_state_*.pt"])
        except Exception as e:  # noqa: BLE001
            logger.warning(f"could not delete previous optimizer states: {e}")
