"""The training engine of one rank: owns the local layers and executes pipeline instructions.

``train_step`` walks the precomputed 1F1B instruction list of this stage (load, receive, forward,
loss, backward, send, tied-gradient reduction, optimizer step) through a dispatch table;
``evaluation_step`` does the same for the fill-drain schedule without gradients;
``run_instructions`` executes ad-hoc lists for inference.  Return records, buffer semantics, loss
averaging (over micro batches and data-parallel ranks) and the shipping of (loss, metrics) from the
last to the first stage follow src/scaling/core/nn/parallel_module/parallel_module.py:92-767.
Unlike the reference, the step has a single host synchronisation (reading the loss), the step time
is measured with CUDA events on the compute stream, and the batch is copied to the device with
non-blocking copies from pinned memory.
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict
from pathlib import Path
from typing import Any, Callable, Generic, NamedTuple, Optional, Union

import torch
import torch.distributed as dist

from ....parallel import fused_tp
from ....parallel.topology import Topology
from ....parallel.topology_config import ActivationCheckpointingType
from ...profiler import Profiler, ProfilerConfig
from ...profiler.timer import CudaEventTimer
from ..parameter_meta import CoreParameterMeta
from ..pipeline_schedule import InstructionBase, PipelineScheduleInference, PipelineScheduleTrain
from .activation_checkpointing import checkpoint
from .base_layer import BaseDatasetBatchGeneric, BaseLossInputGeneric
from .buffers import Buffers, BufferType
from .communicator import PipeCommunicator
from .layer_spec import LayerSpec
from .partitioned_module import PipePartitionedModule


class TrainStepOutput(NamedTuple):
    loss: Optional[float]
    metrics: Optional[dict[str, Union[int, float]]]
    global_grad_norm: Optional[float]
    global_grad_norm_clipped: Optional[float]
    learning_rates: Optional[dict[str, float]]
    overflow: Optional[bool]
    no_overflow_steps: Optional[int]
    current_loss_scale: Optional[float]
    step_duration: float
    debug_dict: Optional[dict[str, float]]


class EvaluationStepOutput(NamedTuple):
    loss: Optional[float]
    metrics: Optional[dict[str, Union[int, float]]]
    step_duration: float


class PipeGrad(NamedTuple):
    tensors: list[torch.Tensor]
    grad_tensors: list[torch.Tensor]


def _to_python(x: Any) -> Any:
    if isinstance(x, dict):
        return {k: _to_python(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_to_python(v) for v in x)
    return x.tolist() if torch.is_tensor(x) else x


def allreduce_tensor_in_float32(tensor: torch.Tensor, process_group: Any) -> None:
    if tensor.dtype == torch.float32:
        dist.all_reduce(tensor, group=process_group)
        return
    f = tensor.float()
    dist.all_reduce(f, group=process_group)
    tensor.copy_(f)


def _broadcast_from_first(tensor: torch.Tensor, process_group: Any) -> None:
    src = dist.get_global_rank(process_group, 0)
    dist.broadcast(tensor.data, src, group=process_group)


_broadcast_parameters = _broadcast_from_first  # name in src/scaling/core/nn/parallel_module/parallel_module.py:765


class ParallelModule(PipePartitionedModule, Generic[BaseLossInputGeneric, BaseDatasetBatchGeneric]):
    def __init__(self, layer_specs: list[LayerSpec], topology: Topology,
                 profiler_config: ProfilerConfig = ProfilerConfig(), use_continuous_recommunication: bool = False):
        super().__init__(layer_specs=layer_specs, topology=topology)
        self.topology: Topology
        t = self.topology
        self.train_schedule = PipelineScheduleTrain(topology=t)
        self.train_instructions: list[InstructionBase] = self.train_schedule.instructions()
        self.train_required_buffer_count = self.train_schedule.required_buffer_count()
        self.evaluation_schedule = PipelineScheduleInference(topology=t)
        self.evaluation_instructions: list[InstructionBase] = self.evaluation_schedule.instructions()
        self.evaluation_required_buffer_count = self.evaluation_schedule.required_buffer_count()
        self.pipe_buffer = Buffers()

        pp = t.config.pipe_parallel_size
        nxt = (t.pipe_parallel_rank + 1) % pp   # wraps around for inference, where the last stage
        prv = (t.pipe_parallel_rank - 1) % pp   # hands its output back to the first
        down, up = t.pipe_down_group, t.pipe_up_group  # activations / gradients travel on separate groups
        self.communicator_in = PipeCommunicator(
            local_device=t.device, recv_grads=False, recv_data=True,
            use_continuous_recommunication=use_continuous_recommunication,
            peer_recv=t.get_global_rank(pipe_parallel_rank=prv) if pp > 1 else None, group=down, grad_group=up,
        )
        self.communicator_out = PipeCommunicator(
            local_device=t.device, recv_grads=True, recv_data=False,
            use_continuous_recommunication=use_continuous_recommunication,
            peer_send=t.get_global_rank(pipe_parallel_rank=nxt) if pp > 1 else None, group=down, grad_group=up,
        )
        self.communicator_loss_in: Optional[PipeCommunicator] = None
        self.communicator_loss_out: Optional[PipeCommunicator] = None
        if pp > 1:
            if t.is_first_pipe_parallel_rank:
                self.communicator_loss_in = PipeCommunicator(
                    local_device=t.device, recv_grads=False, recv_data=True, use_continuous_recommunication=True,
                    peer_recv=t.get_global_rank(pipe_parallel_rank=pp - 1), group=up,
                )
            if t.is_last_pipe_parallel_rank:
                self.communicator_loss_out = PipeCommunicator(
                    local_device=t.device, recv_grads=False, recv_data=False, use_continuous_recommunication=True,
                    peer_send=t.get_global_rank(pipe_parallel_rank=0), group=up,
                )
        self.profiler = Profiler(config=profiler_config, topology=t)
        self.step_timer = CudaEventTimer()
        # receives between pipeline stages are posted ahead of the compute that precedes them (SB200_PIPE_OVERLAP=0:
        # every receive is posted where the schedule names it); a list here records instructions and postings
        self.overlap_pipe_communication = os.environ.get("SB200_PIPE_OVERLAP", "1") != "0"
        self.instruction_trace: Optional[list[str]] = None
        # whole-step CUDA graph (see _graph_eligible); SB200_CUDA_GRAPH=0 disables it
        self.enable_cuda_graph = os.environ.get("SB200_CUDA_GRAPH", "1") != "0"
        self._nvtx = os.environ.get("SB200_NVTX", "0") == "1" and self.topology.device.type == "cuda"
        self._graph: Any = None
        self._graph_failed = False
        self._graph_warmup_left = 2
        self._graph_inputs: list[Any] = []
        self._graph_loss: Any = None
        self._graph_metrics: Optional[dict[str, torch.Tensor]] = None
        self._graph_signature: Any = None
        self._graph_captures = 0
        self._graph_kernel_calls = 0
        self._graph_pending: list[Any] = []
        self._kernel_dropout: Optional[bool] = None
        self._presynced: list[Any] = []
        self._handlers: dict[str, Callable[..., None]] = {
            "LoadMicroBatch": self._do_load, "ForwardPass": self._do_forward, "Loss": self._do_loss,
            "BackwardPass": self._do_backward, "SendActivation": self._do_send_activation,
            "RecvActivation": self._do_recv_activation, "SendGrad": self._do_send_grad,
            "RecvGrad": self._do_recv_grad, "ReduceTiedGrads": self._do_reduce_tied, "StoreMicroBatch": self._do_store,
        }
        self._mark_tied_copies()
        self.broadcast_model()

    def _mark_tied_copies(self) -> None:
        """A tied weight held by this stage whose first owner lives on an earlier stage is a copy: the optimizer
        keeps it in step with the owner (summed gradients, identical update) but counts it once in the gradient norm."""
        tli = self.tied_layer_index
        for local_index, layer in enumerate(self._layers):
            index = self.first_layer_index + local_index
            if tli.layer_index_is_tied_global_duplicate(index) and not tli.layer_index_is_tied_local_duplicate(index):  # type: ignore[union-attr]
                for attr in tli.get_tied_weight_attributes_by_layer_index(index):  # type: ignore[union-attr]
                    target: Any = layer
                    for part in attr.split("."):
                        target = getattr(target, part)
                    target.tied_copy_of_earlier_stage = True

    # ------------------------------------------------------------------ parameters
    def named_parameters_with_meta(self) -> list[tuple[str, torch.Tensor, CoreParameterMeta]]:
        out = []
        for local_index, layer in enumerate(self._layers):
            dup = self.tied_layer_index.layer_index_to_tied_local_duplicate_parameter_names(  # type: ignore[union-attr]
                self.first_layer_index + local_index)
            for name, p in layer.named_parameters():
                if name not in dup:
                    out.append((name, p, p.core_parameter_meta))  # type: ignore[attr-defined]
        return out

    def save_checkpoint(self, dir_: Union[Path, str], separate_file_for_parameters: Optional[list[str]] = None) -> None:
        super().save_checkpoint(dir_=dir_, separate_file_for_parameters=separate_file_for_parameters)
        if self.topology.data_parallel_rank == 0 and self.topology.model_parallel_rank == 0:
            self.save_parameter_meta(Path(dir_))

    def save_parameter_meta(self, dir_: Path) -> None:
        c = self._pipe_partition_coordinates[0]
        out = {}
        for name, _, meta in self.named_parameters_with_meta():
            sd = meta.state_dict()
            sd["local_shape"] = list(sd["local_shape"])
            sd["tied_layer_indices"] = sorted(sd["tied_layer_indices"])
            sd["umup_meta"] = asdict(sd["umup_meta"]) if sd["umup_meta"] else None
            out[f"layer_{meta.layer_index}_{name}"] = sd
        with open(Path(dir_) / f"parameter_meta_{c.start}_{c.end}.json", "w") as f:
            json.dump(out, f, indent=4, default=str)

    def broadcast_model(self) -> None:
        """Make replicas identical: TP-replicated parameters from model rank 0, everything from data rank 0,
        tied copies from the first stage that holds them."""
        t = self.topology
        if not t.is_distributed_initialized:
            return
        for p in self._layers.parameters():
            if p.core_parameter_meta.is_model_parallel_duplicate and t.model_parallel_size > 1:  # type: ignore[attr-defined]
                _broadcast_from_first(p, t.model_parallel_group)
            if t.data_parallel_size > 1:
                _broadcast_from_first(p, t.data_parallel_group)
        for p, group, stages in self.tied_layer_index.local_parameters_and_process_groups():  # type: ignore[union-attr]
            if len(stages) > 1:
                _broadcast_from_first(p, group)

    def umup_setup(self, effective_batch_size: int, depth: int, avg_sequence_length: int,
                   allow_non_umup_params: bool = False) -> None:
        super().umup_setup(effective_batch_size, depth, avg_sequence_length, allow_non_umup_params)
        self.broadcast_model()  # weights were re-drawn

    def get_params_count(self) -> tuple[int, int]:
        """(all parameters over all ranks of one replica, parameters counted once)."""
        t = self.topology
        total = unique = 0
        if t.data_parallel_rank == 0:
            for local_index, layer in enumerate(self._layers):
                tied_dup = self.tied_layer_index.layer_index_is_tied_global_duplicate(  # type: ignore[union-attr]
                    self.first_layer_index + local_index)
                for p in layer.parameters():
                    n = p.nelement()
                    total += n
                    mp_dup = t.model_parallel_rank != 0 and p.core_parameter_meta.is_model_parallel_duplicate  # type: ignore[attr-defined]
                    if not (tied_dup or mp_dup):
                        unique += n
        if t.is_distributed_initialized:
            counts = torch.tensor([total, unique], dtype=torch.int64, device=t.device)
            dist.all_reduce(counts)
            total, unique = (int(v) for v in counts.tolist())
        return total, unique

    # ------------------------------------------------------------------ forward over local layers
    def _forward_tuple_input(self, *args: Any) -> Any:
        x = self._layers[0].tuple_to_input(tuple(args))
        for layer in self._layers:
            x = layer(x)
        return self._layers[-1].output_to_tuple(x)

    def forward(self, x: Any) -> Any:
        mode = self.topology.config.activation_checkpointing_type
        if self.training and torch.is_grad_enabled() and mode == ActivationCheckpointingType.EVERY_PIPE_STAGE:
            out = checkpoint(self._forward_tuple_input, self.topology, *self._layers[0].input_to_tuple(x))
            return self._tuple_to_stage_output(out)
        if self.training and torch.is_grad_enabled() and mode == ActivationCheckpointingType.EVERY_LAYER:
            for i, layer in enumerate(self._layers):
                def run(*args: Any, _layer: Any = layer) -> Any:
                    return _layer.output_to_tuple(_layer(_layer.tuple_to_input(tuple(args))))

                out = checkpoint(run, self.topology, *layer.input_to_tuple(x))
                if i + 1 < len(self._layers):
                    x = self._layers[i + 1].tuple_to_input(out)
                else:
                    x = self._tuple_to_stage_output(out)
            return x
        for layer in self._layers:
            x = layer(x)
        return x

    def _tuple_to_stage_output(self, out: tuple) -> Any:
        last = self._layers[-1]
        if self.topology.is_last_pipe_parallel_rank:
            return last.tuple_to_last_stage_activation(out)
        # an intermediate stage's output is what the first layer of the next stage takes as input
        next_cls = self._layer_specs[self._pipe_partition_coordinates[0].end].module_class
        return next_cls.tuple_to_input(out)

    # ------------------------------------------------------------------ steps
    def _run(self, instructions: list[InstructionBase], **ctx: Any) -> Any:
        optimizer_out = None
        # SB200_NVTX=1: one NVTX range per schedule instruction, for timelines of external profilers
        nvtx = self._nvtx
        post_ahead = self.topology.config.pipe_parallel_size > 1 and self.overlap_pipe_communication
        for position, ins in enumerate(instructions):
            name = ins.name
            if nvtx:
                torch.cuda.nvtx.range_push(f"{name}[mb={ins.micro_batch_id},buf={ins.buffer_id}]")
            try:
                if self.instruction_trace is not None:
                    self.instruction_trace.append(f"{name} mb={ins.micro_batch_id}")
                with self.profiler.time(name, ins.micro_batch_id, ins.buffer_id):
                    if name == "OptimizerStep":
                        optimizer_out = ctx["optimizer"].step()
                    else:
                        self._handlers[name](ins, **ctx)
            finally:
                if nvtx:
                    torch.cuda.nvtx.range_pop()
            if post_ahead:
                self._post_receives_ahead(instructions, position)
        if post_ahead:
            self.communicator_in.drain()
            self.communicator_out.drain()
        return optimizer_out

    def _post_receives_ahead(self, instructions: list[InstructionBase], position: int) -> None:
        """Post the next receive of this step now if only compute lies between here and its instruction, so that the
        transfer runs under that compute (the reference blocks in every receive:
        src/scaling/core/nn/parallel_module/communicator.py:388-482).

        A posted receive is a kernel that waits for the sender.  It must never wait for a send that itself waits,
        through the other stage's schedule, for a send this stage has not issued yet: on a GPU, kernels of different
        streams can share a hardware queue, and the late send could sit behind the waiting receive.  Hence the rule:
        the look-ahead stops at the first send instruction.  Everything the sender needs from this stage is then
        already on its way when the receive is posted.  In the 1F1B schedule this posts the receive of the next
        activation on every stage but the first right after the gradient of the previous micro batch has been sent,
        i.e. under a whole forward and backward pass."""
        for ins in instructions[position + 1:]:
            name = ins.name
            if name in ("SendActivation", "SendGrad"):
                return
            if name == "RecvActivation":
                if self.communicator_in.post_recv() and self.instruction_trace is not None:
                    self.instruction_trace.append(f"post RecvActivation mb={ins.micro_batch_id}")
                return
            if name == "RecvGrad":
                if self.pipe_buffer.has(BufferType.PIPELINE_STAGE_OUTPUT, ins.buffer_id):
                    out = self.pipe_buffer.get(BufferType.PIPELINE_STAGE_OUTPUT, ins.buffer_id)
                    tup = self._prepare_for_send(self._layers[-1].output_to_tuple(out))
                    if self.communicator_out.post_recv_grad(tup) and self.instruction_trace is not None:
                        self.instruction_trace.append(f"post RecvGrad mb={ins.micro_batch_id}")
                return

    # ------------------------------------------------------------------ CUDA-graph training step
    def _graph_eligible(self, optimizer: Any) -> bool:
        """A whole optimizer step (all micro batches, backward, gradient reduction, AdamW, parameter all-gather)
        can be captured once and replayed when nothing in it depends on the host: one pipeline stage (tensor-parallel
        collectives, library or in-kernel, are captured with the rest; the batch is handed to the tensor-parallel
        ranks before the replay), dropout only in the counter-based kernels, no loss
        scaling, profiler idle."""
        if not self.enable_cuda_graph or self._graph_failed:
            return False
        if getattr(self, "_tensor_statistics_active", False):  # hooks of a statistics trace need the eager step
            return False
        t = self.topology
        if t.device.type != "cuda" or t.config.pipe_parallel_size != 1:
            return False
        if not all(hasattr(optimizer, a) for a in ("begin_step", "step_device", "finish_step")):
            return False
        if optimizer.config.loss_scaler.enable or optimizer.config.debug_log:
            return False
        if self.profiler.config.profile_steps > 0:
            return False
        if torch._C._get_tracing_state() is not None:
            return False
        # Dropout is captured when it runs in the counter-based kernels (their seed and step are read from device
        # memory, which the host advances before every replay); torch's generator-based dropout is not.
        for m in self._layers.modules():
            if isinstance(m, torch.nn.Dropout) and m.p > 0.0 and not getattr(m, "kernel_dropout", False):
                return False
            if getattr(m, "dropout_p", 0.0) and m.training and getattr(m, "topology", None) is None:
                return False
        return True

    def _begin_dropout_step(self) -> None:
        """New dropout masks for this step (only where a dropout kernel is active: the update is a small
        host-to-device copy)."""
        if self._kernel_dropout is None:
            self._kernel_dropout = any(
                (isinstance(m, torch.nn.Dropout) and m.p > 0.0 and getattr(m, "kernel_dropout", False))
                or (getattr(m, "dropout_p", 0.0) and getattr(m, "topology", None) is not None)
                for m in self._layers.modules())
        if self._kernel_dropout and self.topology.device.type == "cuda":
            self.topology.kernel_rng.begin_step()

    @staticmethod
    def _batch_tensors(batch: Any) -> list[tuple[str, torch.Tensor]]:
        if isinstance(batch, torch.Tensor):
            return [("", batch)]
        return [(k, v) for k, v in sorted(vars(batch).items()) if isinstance(v, torch.Tensor)]

    def _static_copy(self, batch: Any) -> Any:
        """Device-resident copy of a batch whose tensors keep their addresses for the life of the graph."""
        device = self.topology.device
        if isinstance(batch, torch.Tensor):
            return batch.to(device).clone()
        clone = type(batch).__new__(type(batch))
        clone.__dict__.update(vars(batch))
        for k, v in self._batch_tensors(batch):
            setattr(clone, k, v.to(device).clone())
        return clone

    def _graph_device_step(self, optimizer: Any, sync: Callable, loss_function: Callable,
                           metrics_aggregation_fn: Optional[Callable]) -> None:
        """Device work of one step on the static input batches; runs eagerly for warm-up and under capture."""
        t = self.topology
        self.pipe_buffer.reset()
        fused_tp.begin_step()  # host-side only: the step issues the same fused launches eagerly, captured and replayed
        presynced = t.config.model_parallel_size > 1  # then the static inputs are synchronised batches already
        for batch in self._graph_inputs:
            b = batch if presynced else sync(t, batch)
            out = self(b.only_inputs())
            result = loss_function(out, b.only_targets())
            loss, metrics = result if isinstance(result, tuple) else (result, None)
            self.pipe_buffer.add_loss(loss, metrics)
            optimizer.backward(loss)
        optimizer.step_device()
        total = torch.stack([x.float() for x in self.pipe_buffer.losses]).sum() / t.config.gradient_accumulation_steps
        if t.config.data_parallel_size > 1:
            dist.all_reduce(total, group=t.data_parallel_group)
            total = total / t.config.data_parallel_size
        self._graph_loss.copy_(total)
        if self.pipe_buffer.metrics and metrics_aggregation_fn is not None:
            agg = metrics_aggregation_fn(t, self.pipe_buffer.metrics)
            if self._graph_metrics is None:
                self._graph_metrics = {k: torch.zeros((), dtype=torch.float32, device=t.device) for k in agg}
            for k, v in agg.items():
                self._graph_metrics[k].copy_(torch.as_tensor(v, dtype=torch.float32, device=t.device))

    def cuda_graph_state(self) -> str:
        """How training steps are launched: "whole step" (one captured graph replayed per optimizer step), "eager"
        (instruction list from the host) or "eager (capture failed)"."""
        if self._graph is not None:
            return "whole step"
        return "eager (capture failed)" if self._graph_failed else "eager"

    def release_cuda_graph(self) -> None:
        """Drop the captured training step and its static buffers (call before destroying process groups: a graph
        that holds collectives keeps their communicators busy)."""
        self._graph = None
        self._graph_inputs = []
        self._graph_loss = None
        self._graph_metrics = None
        self._graph_signature = None

    def _graphed_train_step(self, dataloader: Any, optimizer: Any, sync: Callable, loss_function: Callable,
                            metrics_aggregation_fn: Optional[Callable]) -> Optional[TrainStepOutput]:
        """One training step through the captured graph.  Returns None (with the batches it already drew kept in
        ``_graph_pending``) when the step has to run through the instruction list instead."""
        from ....ops import _lib

        t = self.topology
        ga = t.config.gradient_accumulation_steps
        presync = t.config.model_parallel_size > 1
        if presync:
            # The hand-over of a batch to the tensor-parallel ranks reads sizes on the host: it runs here, ahead of
            # the replay, on every rank of the group (only the first one has a data loader); the captured step starts
            # from the synchronised batch.
            raw = [sync(t, next(dataloader) if t.is_io_rank else None) for _ in range(ga)]
        else:
            raw = [next(dataloader) for _ in range(ga)]
        key = (sync, loss_function, metrics_aggregation_fn, presync,
               tuple(tuple((type(b).__name__, k, tuple(v.shape), v.dtype) for k, v in self._batch_tensors(b)) for b in raw))
        if key != self._graph_signature:
            # new input signature: drop the old graph and start over (a bounded number of times)
            self._graph = None
            self._graph_captures += 1
            if self._graph_captures > 4:
                self._graph_failed = True
                if presync:
                    self._presynced = raw
                else:
                    self._graph_pending = raw
                return None
            self._graph_signature = key
            self._graph_warmup_left = 2 if self._graph_captures == 1 else 1
            self._graph_inputs = [self._static_copy(b) for b in raw]
            self._graph_loss = torch.zeros((), dtype=torch.float32, device=t.device)
            self._graph_metrics = None
        else:
            for static, b in zip(self._graph_inputs, raw):
                if isinstance(static, torch.Tensor):
                    static.copy_(b, non_blocking=True)
                    continue
                for k, v in self._batch_tensors(b):
                    getattr(static, k).copy_(v, non_blocking=True)
        optimizer.begin_step()
        if self._graph is None:
            self._graph_warmup_left -= 1
            if self._graph_warmup_left >= 0:
                # the first steps run eagerly: lazy initialisation (kernel attributes, NCCL, allocator) must not
                # happen under capture
                self._graph_device_step(optimizer, sync, loss_function, metrics_aggregation_fn)
            else:
                try:
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    calls0 = _lib.kernel_calls()
                    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                        self._graph_device_step(optimizer, sync, loss_function, metrics_aggregation_fn)
                    self._graph_kernel_calls = _lib.kernel_calls() - calls0
                    self._graph = graph
                    failed = None
                except Exception as e:  # noqa: BLE001 - any capture problem means: stay eager
                    failed = e
                    self._graph = None
                # Ranks decide together: a step holds collectives, so either every rank replays it or none does.
                if t.is_distributed_initialized and t.world_size > 1:
                    flag = torch.tensor([0.0 if failed is None else 1.0], device=t.device)
                    dist.all_reduce(flag)
                    if flag.item() > 0 and failed is None:
                        failed = RuntimeError("capture failed on another rank")
                        self._graph = None
                if failed is not None:
                    from ...logging import logger

                    logger.warning(f"CUDA-graph capture of the training step failed ({type(failed).__name__}: {failed}); "
                                   "continuing without graphs")
                    self._graph_failed = True
                    torch.cuda.synchronize()
                    optimizer.zero_grad()
                    self._graph_device_step(optimizer, sync, loss_function, metrics_aggregation_fn)
                else:
                    self._graph.replay()
        else:
            self._graph.replay()
            _lib.note_replayed_calls(self._graph_kernel_calls)
        opt_out = optimizer.finish_step()
        loss = float(self._graph_loss.item())
        metrics = None if self._graph_metrics is None else {k: v.item() for k, v in self._graph_metrics.items()}
        self.step_timer.stop()
        return TrainStepOutput(loss=loss, metrics=metrics, step_duration=self.step_timer.duration(), **opt_out._asdict())

    def train_step(self, dataloader: Any, optimizer: Any, sync_batch_to_model_parallel: Callable,
                   loss_function: Callable, metrics_aggregation_fn: Optional[Callable] = None) -> TrainStepOutput:
        if not torch.is_grad_enabled():
            raise RuntimeError("train_step() requires gradients enabled. Use evaluation_step() instead.")
        self.step_timer.start()
        self._begin_dropout_step()
        if self._graph_eligible(optimizer):
            self._layers.train()
            out = self._graphed_train_step(dataloader, optimizer, sync_batch_to_model_parallel, loss_function,
                                           metrics_aggregation_fn)
            if out is not None:
                return out
            if self._graph_pending:
                import itertools

                dataloader, self._graph_pending = itertools.chain(self._graph_pending, dataloader), []
        self._layers.train()
        self._set_channel("train")
        self.pipe_buffer.reset()
        fused_tp.begin_step()
        self.profiler.step()
        opt_out = self._run(self.train_instructions, dataloader=dataloader, optimizer=optimizer,
                            sync=sync_batch_to_model_parallel, loss_function=loss_function, grad=True)
        loss, metrics = self.get_loss(metrics_aggregation_fn)
        self.step_timer.stop()
        self.profiler.flush()
        return TrainStepOutput(loss=loss, metrics=metrics, step_duration=self.step_timer.duration(), **opt_out._asdict())

    def evaluation_step(self, dataloader: Any, sync_batch_to_model_parallel: Callable, loss_function: Callable,
                        metrics_aggregation_fn: Optional[Callable] = None) -> EvaluationStepOutput:
        self.step_timer.start()
        self._layers.eval()
        self._set_channel("eval")
        self.pipe_buffer.reset()
        fused_tp.begin_step()
        self.profiler.step()
        with torch.no_grad():
            self._run(self.evaluation_instructions, dataloader=dataloader, optimizer=None,
                      sync=sync_batch_to_model_parallel, loss_function=loss_function, grad=False)
        loss, metrics = self.get_loss(metrics_aggregation_fn)
        self.step_timer.stop()
        self.profiler.flush()
        return EvaluationStepOutput(loss=loss, metrics=metrics, step_duration=self.step_timer.duration())

    def run_instructions(self, instructions: list[InstructionBase], sync_batch_to_model_parallel: Callable,
                         collect_outputs_from_model_parallel: Callable, batch: Any = None) -> Any:
        for ins in instructions:
            if ins.name not in ("StoreMicroBatch", "ForwardPass", "SendActivation", "RecvActivation"):
                raise NotImplementedError(f"Instruction '{ins.name}' not implemented for run_instructions.")
            self._handlers[ins.name](ins, sync=sync_batch_to_model_parallel, batch=batch, take_input=True)
        t = self.topology
        if not instructions:
            return None
        last = instructions[-1]
        if batch is not None and t.config.pipe_parallel_size == 1:
            out = self.pipe_buffer.take(BufferType.PIPELINE_STAGE_OUTPUT, last.buffer_id)
            return collect_outputs_from_model_parallel(t, out)
        if t.config.pipe_parallel_size > 1 and t.pipe_parallel_rank == 0 and last.name == "RecvActivation":
            out = self.pipe_buffer.take(BufferType.PIPELINE_STAGE_INPUT, last.buffer_id)
            return collect_outputs_from_model_parallel(t, out)
        return None

    def get_loss(self, metrics_aggregation_fn: Optional[Callable]) -> tuple[Optional[float], Optional[dict]]:
        t = self.topology
        data = None
        if t.is_last_pipe_parallel_rank:
            losses = self.pipe_buffer.losses
            assert losses, "no loss was recorded in this step"
            loss = torch.stack([x.float() for x in losses]).sum() / t.config.gradient_accumulation_steps
            metrics = None
            if self.pipe_buffer.metrics:
                assert metrics_aggregation_fn is not None
                metrics = metrics_aggregation_fn(t, self.pipe_buffer.metrics)
            if t.config.data_parallel_size > 1:
                dist.all_reduce(loss, group=t.data_parallel_group)
                loss = loss / t.config.data_parallel_size
            data = (loss, metrics)
        if t.config.pipe_parallel_size > 1:
            if t.is_last_pipe_parallel_rank:
                assert self.communicator_loss_out is not None
                self.communicator_loss_out.send_data(data)
                self.communicator_loss_out.drain()
                return None, None
            if t.is_first_pipe_parallel_rank:
                assert self.communicator_loss_in is not None
                loss, metrics = self.communicator_loss_in.recv_data()
                return float(loss.item()), _to_python(metrics)
            return None, None
        loss, metrics = data  # type: ignore[misc]
        return float(loss.item()), _to_python(metrics)

    # ------------------------------------------------------------------ instruction handlers
    def _do_store(self, ins: InstructionBase, sync: Callable, batch: Any = None, **_: Any) -> None:
        self.pipe_buffer.write(BufferType.PIPELINE_STAGE_INPUT, ins.buffer_id, sync(self.topology, batch))

    def _do_load(self, ins: InstructionBase, dataloader: Any, sync: Callable, **_: Any) -> None:
        t = self.topology
        if self._presynced:  # batches that a step drew and synchronised before it fell back to this path
            batch = self._presynced.pop(0)
        else:
            batch = None
            if t.is_io_rank:
                assert dataloader is not None
                batch = next(dataloader)
            batch = sync(t, batch)
        if t.is_first_pipe_parallel_rank:
            self.pipe_buffer.write(BufferType.PIPELINE_STAGE_INPUT, ins.buffer_id, batch.only_inputs())
        if t.is_last_pipe_parallel_rank:
            self.pipe_buffer.write(BufferType.TARGET, ins.buffer_id, batch.only_targets())

    def _do_forward(self, ins: InstructionBase, take_input: bool = False, **_: Any) -> None:
        op = self.pipe_buffer.take if take_input else self.pipe_buffer.get
        x = op(BufferType.PIPELINE_STAGE_INPUT, ins.buffer_id)
        self.pipe_buffer.write(BufferType.PIPELINE_STAGE_OUTPUT, ins.buffer_id, self(x))

    def _do_loss(self, ins: InstructionBase, loss_function: Callable, **_: Any) -> None:
        out = self.pipe_buffer.get(BufferType.PIPELINE_STAGE_OUTPUT, ins.buffer_id)
        first_pass = True if ins.is_first_pass is None else ins.is_first_pass
        target = (self.pipe_buffer.get if first_pass else self.pipe_buffer.take)(BufferType.TARGET, ins.buffer_id)
        result = loss_function(out, target)
        loss, metrics = result if isinstance(result, tuple) else (result, None)
        assert torch.is_tensor(loss) and loss.dim() == 0, (
            f"The loss needs to be a scalar. The loss currently has the shape: {getattr(loss, 'shape', None)}"
        )
        self.pipe_buffer.add_loss(loss, metrics)
        self.pipe_buffer.write(BufferType.LOSS, ins.buffer_id, loss)

    def _do_backward(self, ins: InstructionBase, optimizer: Any, **_: Any) -> None:
        if self.topology.is_last_pipe_parallel_rank:
            optimizer.backward(self.pipe_buffer.take(BufferType.LOSS, ins.buffer_id))
            self.pipe_buffer.dump(BufferType.PIPELINE_STAGE_OUTPUT, ins.buffer_id)
            self.pipe_buffer.dump(BufferType.TARGET, ins.buffer_id)
        else:
            g: PipeGrad = self.pipe_buffer.take(BufferType.GRAD, ins.buffer_id)
            torch.autograd.backward(tensors=g.tensors, grad_tensors=g.grad_tensors)
        if self.topology.is_first_pipe_parallel_rank:
            self.pipe_buffer.dump(BufferType.PIPELINE_STAGE_INPUT, ins.buffer_id)

    def _do_send_activation(self, ins: InstructionBase, **_: Any) -> None:
        out = self.pipe_buffer.get(BufferType.PIPELINE_STAGE_OUTPUT, ins.buffer_id)
        self.communicator_out.send_data(self._prepare_for_send(self._layers[-1].output_to_tuple(out)))

    def _do_recv_activation(self, ins: InstructionBase, **_: Any) -> None:
        tup = self._after_recv(self.communicator_in.recv_data())
        first = self._layers[0]
        x = first.tuple_to_last_stage_activation(tup) if self.topology.is_first_pipe_parallel_rank else first.tuple_to_input(tup)
        self.pipe_buffer.write(BufferType.PIPELINE_STAGE_INPUT, ins.buffer_id, x)

    def _do_send_grad(self, ins: InstructionBase, **_: Any) -> None:
        x = self.pipe_buffer.take(BufferType.PIPELINE_STAGE_INPUT, ins.buffer_id)
        self.communicator_in.send_grad(self._layers[0].input_to_tuple(x))

    def _do_recv_grad(self, ins: InstructionBase, **_: Any) -> None:
        out = self.pipe_buffer.take(BufferType.PIPELINE_STAGE_OUTPUT, ins.buffer_id)
        tensors, grads = self.communicator_out.recv_grad(self._prepare_for_send(self._layers[-1].output_to_tuple(out)))
        self.pipe_buffer.write(BufferType.GRAD, ins.buffer_id, PipeGrad(tensors, grads))

    def _do_reduce_tied(self, ins: InstructionBase, **_: Any) -> None:
        for p, group, stages in self.tied_layer_index.local_parameters_and_process_groups():  # type: ignore[union-attr]
            if len(stages) > 1 and p.grad is not None:
                allreduce_tensor_in_float32(p.grad, group)
        if self.topology.config.model_parallel_size > 1:
            for p in self._layers.parameters():
                if p.core_parameter_meta.tied_grad_on_model_parallel and p.grad is not None:  # type: ignore[attr-defined]
                    allreduce_tensor_in_float32(p.grad, self.topology.model_parallel_group)

    # hooks for subclasses that strip / rebuild variable-shape fields around the pipe transfer
    def _prepare_for_send(self, tup: tuple) -> tuple:
        return tup

    def _after_recv(self, tup: tuple) -> tuple:
        return tup

    def _set_channel(self, channel: str) -> None:
        """Training and evaluation steps negotiate the structure of what crosses a stage boundary separately."""
        for c in (self.communicator_in, self.communicator_out, self.communicator_loss_in, self.communicator_loss_out):
            if c is not None:
                c.channel = channel

    def reset_activation_shape(self) -> None:
        """Forget negotiated shapes; must be called on all ranks together."""
        for c in (self.communicator_in, self.communicator_out, self.communicator_loss_in, self.communicator_loss_out):
            if c is not None:
                c.reset_communication_meta()
