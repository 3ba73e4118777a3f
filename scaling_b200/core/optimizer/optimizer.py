"""Mixed-precision AdamW with data-parallel gradient reduction and ZeRO stage 1.

One step (reference semantics: src/scaling/core/optimizer/optimizer.py:114-215, its helpers in
parameter_group.py:351-540 and allreduce.py:16-66), re-organised so that nothing but two scalars
ever reaches the host:

  1. tensor-parallel all-reduce of the gradients that are partial per rank (one slice per group);
  2. data-parallel reduction of the flat gradient buffer - reduce-scatter with ZeRO (each rank
     receives only the range it owns), all-reduce otherwise;
  3. sum of squares of the reduced gradients plus a sticky inf/nan flag (one kernel per range), summed
     over all ranks in ONE two-float all-reduce - this replaces the reference's per-parameter host
     synchronisations for the overflow check and its separate TP / PP norm reductions;
  4. the gradient multiplier ``1 / (dp * loss_scale) * clip_coefficient`` and the skip flag are
     computed on the device and consumed by the fused AdamW kernel, which updates the fp32 master
     weights and moments and writes the low-precision parameters in the same pass;
  5. with ZeRO, an all-gather of the updated parameter ranges (in place in the flat buffer);
  6. one memset clears the gradient buffer.

Checkpoints are layout independent and use the reference's file format: one
``optimizer_state_layer_{i}.pt`` per layer holding, per parameter key, the tensor-parallel-merged
fp32 master weight and Adam moments (``optimizer.py:342-455``), or raw per-rank files with
``zero_save_static``.
"""

from __future__ import annotations

import collections
from pathlib import Path
from typing import Any, List, Optional, Union

import torch
import torch.distributed as dist

from ...ops import functional as K
from ...ops._lib import CommTimeout
from ...parallel.topology import Topology
from ..logging import logger
from ..nn.parameter_meta import CoreParameterMeta
from ..utils.param_merge import merge_parameter, split_parameter
from .base import BaseOptimizer, OptimizerStepOutput
from .learning_rate_scheduler import LearningRateSchedulerConfig
from .loss_scaler import LossScaler
from .optimizer_config import OptimizerConfig, OptimizerParamGroupConfig
from .parameter_group import OptimizerParamGroup


def get_new_optimizer_groups_by_lr_gain_per_param(parameter_groups: List[OptimizerParamGroup],
                                                  topology: Topology) -> List[OptimizerParamGroup]:
    """Split every group by the per-parameter learning-rate gain (u-muP); all pipeline stages agree
    on the set of gains so that the same groups exist everywhere (possibly empty)."""
    out: List[OptimizerParamGroup] = []
    for group in parameter_groups:
        gains = {m.lr_gain for m in group.parameter_metas}
        if topology.config.pipe_parallel_size > 1 and topology.is_distributed_initialized:
            gathered: list[Any] = [None] * topology.config.pipe_parallel_size
            dist.all_gather_object(gathered, gains, group=topology.pipe_parallel_group)
            gains = set().union(*gathered)
        if not gains:
            gains = {1.0}
        base = group.config.learning_rate_scheduler
        for gain in sorted(gains):
            lr_cfg = LearningRateSchedulerConfig(
                learning_rate=gain * base.learning_rate,
                learning_rate_minimum=gain * base.learning_rate_minimum,
                learning_rate_decay_style=base.learning_rate_decay_style,
                learning_rate_decay_iters=base.learning_rate_decay_iters,
                learning_rate_warmup_steps=base.learning_rate_warmup_steps,
                learning_rate_warmup_delay_steps=base.learning_rate_warmup_delay_steps,
            )
            members = [
                (n, p, m) for n, p, m in zip(group.parameter_names, group.parameters_original, group.parameter_metas)
                if m.lr_gain == gain
            ]
            out.append(OptimizerParamGroup(
                named_parameters_with_meta=members,
                config=OptimizerParamGroupConfig(
                    name=f"{group.config.name}_lr_gain_{gain}", learning_rate_scheduler=lr_cfg,
                    weight_decay=group.config.weight_decay,
                    independent_weight_decay=group.config.independent_weight_decay,
                ),
            ))
    return out


class Optimizer(BaseOptimizer):
    def __init__(self, config: OptimizerConfig, parameter_groups: List[OptimizerParamGroup], topology: Topology,
                 scale_backward_by_grad_acc: bool = True) -> None:
        super().__init__(config)
        self.config: OptimizerConfig = config
        if config.method != "adamw":
            raise ValueError(f"Unknown optimization method: {config.method}.")
        self.topology = topology
        self.parameter_groups = get_new_optimizer_groups_by_lr_gain_per_param(parameter_groups, topology)
        self._assert_no_parameter_duplicates()
        for g in self.parameter_groups:
            g.initialize(topology=topology, zero=config.zero)
        self.step_index = 0
        self.adam_steps = 0  # updates actually applied (bias correction); skipped steps do not count
        self.loss_scaler = LossScaler(config=config.loss_scaler)
        self.scale_backward_by_grad_acc = scale_backward_by_grad_acc
        dev = topology.device
        self._stats = torch.zeros(3, dtype=torch.float32, device=dev)     # [sum of squares, overflows, waits given up]
        self._flag = torch.zeros(1, dtype=torch.int32, device=dev)
        self._control = torch.zeros(2, dtype=torch.float32, device=dev)   # [gradient multiplier, skip]
        # read by the host once per step: [global norm, skip, a device-side wait gave up, norm after clipping]
        self._result = torch.zeros(4, dtype=torch.float32, device=dev)
        self._hyper_host: Optional[torch.Tensor] = None                    # [lr, 1-b1^t, 1-b2^t] per group (pinned)
        self._hyper: Optional[torch.Tensor] = None
        self._learning_rates: dict[str, float] = {}
        self._debug = None
        self._slot_variable_names = ["exp_avg", "exp_avg_sq"]
        self._fused = None
        if config.fused_collectives and config.zero and topology.config.data_parallel_size > 1 and dev.type == "cuda":
            self._fused = _try_fused_zero(self)

    def _assert_no_parameter_duplicates(self) -> None:
        seen: collections.Counter = collections.Counter()
        names = {}
        for g in self.parameter_groups:
            for n, p in zip(g.parameter_names, g.parameters_original):
                seen[id(p)] += 1
                names[id(p)] = n
        dup = [names[i] for i, c in seen.items() if c > 1]
        assert not dup, (
            f"parameters occurring more than once: {dup}; careful layer indices are relative to pipeline rank, "
            f"this is pipe_parallel_rank {self.topology.pipe_parallel_rank}"
        )

    # ------------------------------------------------------------------ backward / step
    @property
    def data_parallel_exchange(self) -> str:
        """How gradients and parameters cross the data-parallel group: "none", "nccl", "p2p" or "p2p+multicast"."""
        if self.topology.config.data_parallel_size <= 1:
            return "none"
        if self._fused is None:
            return "nccl"
        return "p2p+multicast" if self._fused.use_multicast else "p2p"

    def zero_grad(self, set_to_none: bool = True) -> None:
        for g in self.parameter_groups:
            g.zero_grad(set_to_none)

    def backward(self, loss: torch.Tensor) -> None:
        loss = loss.float()
        ga = self.topology.config.gradient_accumulation_steps
        if ga > 1 and self.scale_backward_by_grad_acc:
            loss = loss / ga
        self.loss_scaler.scale_loss(loss).backward()

    def _reduce_gradients(self, g: OptimizerParamGroup) -> torch.Tensor:
        """Reduce over tensor-parallel (partial-gradient slice) and data-parallel ranks; returns the
        reduced gradient of the owned range (still scaled by dp * loss_scale)."""
        t = self.topology
        a, b = g.segment_ends[1], g.segment_ends[2]
        if b > a and t.config.model_parallel_size > 1:
            dist.all_reduce(g.flat_grad[a:b], group=t.model_parallel_group)
        dp = t.config.data_parallel_size
        if dp == 1:
            return g.flat_grad
        group = t.data_parallel_group
        if not g.zero:
            dist.all_reduce(g.flat_grad, group=group)
            return g.flat_grad
        assert g.reduced_grad is not None
        if dist.get_backend(group) == "gloo":  # no reduce-scatter in gloo
            dist.all_reduce(g.flat_grad, group=group)
            lo, hi = g.owned_range
            g.reduced_grad.copy_(g.flat_grad[lo:hi])
        else:
            dist.reduce_scatter_tensor(g.reduced_grad, g.flat_grad, group=group)
        return g.reduced_grad

    def step(self) -> OptimizerStepOutput:
        self.begin_step()
        self.step_device()
        return self.finish_step()

    # The step is split in three so that the device part can live inside a captured CUDA graph:
    # begin_step (host: counters, learning rates -> device), step_device (kernels and collectives only),
    # finish_step (host: the step's single device -> host read, loss-scaler state machine).
    def begin_step(self) -> None:
        self.step_index += 1
        cfg = self.config
        values = []
        self._learning_rates = {}
        for i, g in enumerate(self.parameter_groups):
            lr = g.set_learning_rate(self.step_index)
            self._learning_rates[g.config.name or f"parameter_group_{i}"] = lr
            for _, _, born in g.step_ranges:
                # Parameters whose moments started later than the others (added adapters next to restored weights)
                # count their own updates, as torch's per-parameter ``state['step']`` does
                # (src/scaling/core/optimizer/optimizer.py keeps ``step`` per parameter in its checkpoints).
                t = self.adam_steps + 1 - born
                values += [lr, 1.0 - cfg.beta1 ** t, 1.0 - cfg.beta2 ** t]
        if self._hyper_host is None or self._hyper_host.numel() != len(values):
            self._hyper_host = torch.empty(len(values), dtype=torch.float32,
                                           pin_memory=self.topology.device.type == "cuda")
            self._hyper = torch.empty(len(values), dtype=torch.float32, device=self.topology.device)
        self._hyper_host.copy_(torch.tensor(values, dtype=torch.float32))
        self._hyper.copy_(self._hyper_host, non_blocking=True)
        self._debug = self._debug_norms() if cfg.debug_log else None

    def step_device(self) -> None:
        t = self.topology
        dp = t.config.data_parallel_size
        cfg = self.config
        self._stats.zero_()
        self._flag.zero_()
        if self._fused is not None:
            reduced = self._fused.reduce_scatter(self)
        else:
            reduced = [self._reduce_gradients(g) for g in self.parameter_groups]
        for g, r in zip(self.parameter_groups, reduced):
            for a, b in g.norm_ranges(t):
                K.sumsq_(r[a:b], self._stats[0:1], self._flag, 1.0, True)
        # The overflow flag and the status word of the kernels with bounded waits (peer barriers, fused tensor-parallel
        # GEMMs) travel with the sum of squares: one all-reduce makes every rank agree on norm, overflow and on
        # whether some rank's wait gave up, in which case all of them skip the update.
        K.step_control(0, self._stats, self._flag, self._control, self._result)
        replicas = 1.0
        if t.is_distributed_initialized and t.world_size > 1:
            dist.all_reduce(self._stats)
            if not cfg.zero and dp > 1:
                replicas = float(dp)  # replicas hold identical gradients: count them once
        K.step_control(1, self._stats, self._flag, self._control, self._result,
                       inv=1.0 / (dp * self.loss_scaler.current_scale), clip=float(cfg.gradient_clipping),
                       replicas=replicas)
        slot = 0
        for g, r in zip(self.parameter_groups, reduced):
            lo, hi = g.owned_range
            grad = r if r.numel() == g.master.numel() else r[lo:hi]
            for a, b, born in g.step_ranges:  # one launch per range of equal age: one, but for the case above
                a, b = max(a, lo) - lo, min(b, hi) - lo
                if b > a:
                    p_lp = None if g.dtype == torch.float32 else g.flat_param[lo + a:lo + b]
                    K.adamw_step(g.master[a:b], g.exp_avg[a:b], g.exp_avg_sq[a:b], grad[a:b], p_lp, g.current_lr,
                                 cfg.beta1, cfg.beta2, cfg.eps, g.weight_decay, self.adam_steps + 1 - born,
                                 self._control, self._hyper[3 * slot:3 * slot + 3])
                slot += 1
        if self._fused is not None:
            self._fused.all_gather(self)
        elif cfg.zero and dp > 1:
            for g in self.parameter_groups:
                lo, hi = g.owned_range
                grp = t.data_parallel_group
                if dist.get_backend(grp) == "gloo":
                    parts = [torch.empty_like(g.flat_param[lo:hi]) for _ in range(dp)]
                    dist.all_gather(parts, g.flat_param[lo:hi].contiguous(), group=grp)
                    g.flat_param.copy_(torch.cat(parts))
                else:
                    dist.all_gather_into_tensor(g.flat_param, g.flat_param[lo:hi], group=grp)
        self.zero_grad()
        if self._result.is_cuda:  # a wait of the parameter exchange that gave up after the statistics were taken
            K.step_control(2, self._stats, self._flag, self._control, self._result)

    def finish_step(self) -> OptimizerStepOutput:
        cfg = self.config
        # the only device -> host transfer of the step
        norm_host, bad_host, timed_out, clipped_host = self._result.tolist()
        if timed_out:
            # Some rank's kernel stopped waiting for a peer (SB200_P2P_TIMEOUT_S): its result is incomplete.  Every
            # rank skipped the update (the flag was summed over the ranks before AdamW ran) unless the wait that gave
            # up was the parameter exchange after it; either way the replicas can no longer be trusted to agree.
            K.status_word().zero_()
            raise CommTimeout(
                f"optimizer step {self.step_index}: a device-side wait on a peer gave up (a rank arrived more than "
                "SB200_P2P_TIMEOUT_S late or has left); the step was skipped - resume from the last checkpoint"
            )
        overflow = bool(bad_host)
        scaler_out = self.loss_scaler.step(overflow)
        if overflow:
            if not cfg.loss_scaler.enable:
                raise RuntimeError(
                    f"the global gradient norm is not finite ({norm_host}); enable the loss scaler for fp16 training "
                    "or inspect the gradients with optimizer.debug_log"
                )
            logger.warning("loss scaler encountered overflow, skipping step")
            return OptimizerStepOutput(None, None, None, True, scaler_out.no_overflow_steps,
                                       scaler_out.current_loss_scale, None)
        self.adam_steps += 1
        return OptimizerStepOutput(
            global_grad_norm=norm_host, global_grad_norm_clipped=clipped_host, learning_rates=dict(self._learning_rates),
            overflow=scaler_out.overflow, no_overflow_steps=scaler_out.no_overflow_steps,
            current_loss_scale=scaler_out.current_loss_scale, debug_dict=self._debug,
        )

    def _debug_norms(self) -> dict[str, float]:
        out = {}
        for g in self.parameter_groups:
            for p, m in zip(g.parameters_original, g.parameter_metas):
                name = f"{m.parameter_name}-layer-{m.layer_index}"
                if p.grad is not None:
                    out[f"debug/{name}-grad-norm"] = float(p.grad.float().norm().item())
                out[f"debug/{name}-norm"] = float(p.float().norm().item())
                out[f"debug/{name}-pct-zero"] = 1.0 - float((p.count_nonzero() / max(p.numel(), 1)).item())
        return out

    def refresh_optimizer_after_model_change(self) -> None:
        for g in self.parameter_groups:
            g.refresh_optimized_params(self.topology)

    def log_state(self) -> None:
        for g in self.parameter_groups:
            logger.info(f"optimizer group {g.config.name}: {len(g.parameters_original)} parameters, "
                        f"{g.numel} elements, zero={g.zero}")

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict[str, Any]:
        return {
            "step_index": self.step_index,
            "adam_steps": self.adam_steps,
            "parameter_groups": [g.state_dict() for g in self.parameter_groups],
            "loss_scaler": self.loss_scaler.state_dict(),
        }

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self.step_index = state["step_index"]
        self.adam_steps = state.get("adam_steps", self.step_index)
        self.loss_scaler.load_state_dict(state["loss_scaler"])
        for g, s in zip(self.parameter_groups, state["parameter_groups"]):
            g.load_state_dict(s)

    def _static_file(self, directory: Path) -> Path:
        t = self.topology
        return directory / (f"optimizer_state_static_mp_{t.model_parallel_rank}_pp_{t.pipe_parallel_rank}_"
                            f"dp_{t.data_parallel_rank}.pt")

    def _full_state(self, g: OptimizerParamGroup, tensor: torch.Tensor) -> torch.Tensor:
        """The state tensor for the whole flat buffer (ZeRO: gathered from all data-parallel ranks)."""
        if not g.zero or self.topology.config.data_parallel_size == 1:
            return tensor
        dp = self.topology.config.data_parallel_size
        parts = [torch.empty_like(tensor) for _ in range(dp)]
        dist.all_gather(parts, tensor.contiguous(), group=self.topology.data_parallel_group)
        return torch.cat(parts)

    def _param_groups_for_checkpoint(self) -> list[dict[str, Any]]:
        return [
            {"lr": g.current_lr, "weight_decay": g.weight_decay, "betas": (self.config.beta1, self.config.beta2),
             "eps": self.config.eps, "name": g.config.name, "params": []}
            for g in self.parameter_groups
        ]

    def save_checkpoint(self, directory: Union[Path, str]) -> None:
        t = self.topology
        directory = Path(directory)
        if t.data_parallel_rank != 0 and not self.config.zero:
            return
        directory.mkdir(parents=True, exist_ok=True)
        if self.config.zero and self.config.zero_save_static:
            torch.save(self.state_dict(), str(self._static_file(directory)))
            return
        per_layer: dict[int, dict[str, Any]] = {}
        for g in self.parameter_groups:
            master = self._full_state(g, g.master)
            m1 = self._full_state(g, g.exp_avg)
            m2 = self._full_state(g, g.exp_avg_sq)
            if t.data_parallel_rank != 0:
                continue  # took part in the gather; data-parallel rank 0 of each column writes
            for (a, b), p, meta in zip(g.param_slices(), g.parameters_original, g.parameter_metas):
                shape = p.shape
                merged = merge_parameter(master[a:b].view(shape), meta, t)
                merged_meta = CoreParameterMeta(
                    local_shape=tuple(merged.shape), is_model_parallel=meta.is_model_parallel,
                    model_parallel_dimension=meta.model_parallel_dimension, layer_index=meta.layer_index,
                    parameter_name=meta.parameter_name, layer_class_name=meta.layer_class_name, is_tied=meta.is_tied,
                    tied_layer_indices=set(meta.tied_layer_indices),
                )
                entry = {
                    "parameter": merged,
                    "meta": merged_meta.state_dict(),
                    "optimizer_state": {
                        "step": torch.tensor(float(self.adam_steps - g.born_at(a))),
                        "exp_avg": merge_parameter(m1[a:b].view(shape), meta, t),
                        "exp_avg_sq": merge_parameter(m2[a:b].view(shape), meta, t),
                    },
                }
                layers = {meta.layer_index} | (set(meta.tied_layer_indices) if meta.is_tied else set())
                for li in layers:
                    per_layer.setdefault(li, {})[meta.key_for_layer(li) if meta.is_tied else meta.key] = entry
        if t.data_parallel_rank == 0 and t.model_parallel_rank == 0:
            for li, params in per_layer.items():
                torch.save(
                    {"step_index": self.step_index, "loss_scaler": self.loss_scaler.state_dict(),
                     "parameters": params, "optimizer_param_groups": self._param_groups_for_checkpoint()},
                    str(directory / f"optimizer_state_layer_{li}.pt"),
                )

    def load_checkpoint(self, directory: Union[Path, str]) -> None:
        t = self.topology
        directory = Path(directory)
        static = self._static_file(directory)
        if self.config.zero and self.config.zero_save_static and static.is_file():
            self.load_state_dict(torch.load(str(static), map_location="cpu", weights_only=False))
            return
        cache: dict[int, Optional[dict[str, Any]]] = {}

        def layer_file(li: int) -> Optional[dict[str, Any]]:
            if li not in cache:
                f = directory / f"optimizer_state_layer_{li}.pt"
                cache[li] = torch.load(str(f), map_location="cpu", weights_only=False) if f.is_file() else None
            return cache[li]

        loaded_any = False
        steps: list[list[int]] = []
        for g in self.parameter_groups:
            lo, hi = g.owned_range
            steps.append([0] * len(g.parameters_original))
            # assemble the full-buffer fp32 states on the host, then keep the owned range
            full = {k: torch.zeros(g.padded_numel, dtype=torch.float32) for k in ("parameter", "exp_avg", "exp_avg_sq")}
            full["parameter"].copy_(g.flat_param.float().cpu())
            for pi, ((a, b), p, meta) in enumerate(zip(g.param_slices(), g.parameters_original, g.parameter_metas)):
                entry = None
                candidates = sorted(meta.tied_layer_indices) if meta.is_tied else [meta.layer_index]
                for li in candidates:
                    data = layer_file(li)
                    if data is None:
                        continue
                    keys = [k for k in meta.possible_keys() if k in data["parameters"]]
                    if not keys:
                        # The same weight can be sharded in one layout and replicated in another (KV projections of
                        # multi-query attention are replicated once the group outgrows the KV heads): its key then
                        # differs in the parallel flags only.  The stored tensors are always the complete weight.
                        stem = f"layer_index_{li}_parameter_name_{meta.parameter_name}_is_model_parallel_"
                        keys = [k for k in data["parameters"] if k.startswith(stem)]
                    for key in keys[:1]:
                        if key in data["parameters"]:
                            entry = data["parameters"][key]
                            self.step_index = data["step_index"]
                            steps[-1][pi] = int(entry["optimizer_state"]["step"])
                            self.loss_scaler.load_state_dict(data["loss_scaler"])
                            break
                    if entry is not None:
                        break
                if entry is None:
                    logger.warning(f"no optimizer state found for {meta.key}: it starts from zero moments and counts "
                                   "its own updates for the bias correction")
                    continue
                loaded_any = True
                tensors = {"parameter": entry["parameter"], "exp_avg": entry["optimizer_state"]["exp_avg"],
                           "exp_avg_sq": entry["optimizer_state"]["exp_avg_sq"]}
                for k, v in tensors.items():
                    v = v.float()
                    if meta.is_model_parallel and t.config.model_parallel_size > 1:
                        v = split_parameter(v, meta, t)
                    full[k][a:b].copy_(v.reshape(-1))
            g.master.copy_(full["parameter"][lo:hi])
            g.exp_avg.copy_(full["exp_avg"][lo:hi])
            g.exp_avg_sq.copy_(full["exp_avg_sq"][lo:hi])
        if not loaded_any:
            logger.warning(f"no optimizer state files found in {directory}")
            return
        # The optimizer's counter is the oldest parameter's; younger ones (no stored state: step 0) keep the difference.
        self.adam_steps = max(max(s, default=0) for s in steps)
        for g, s in zip(self.parameter_groups, steps):
            g.set_parameter_steps([self.adam_steps - v for v in s])
        self._hyper_host = None  # the number of ranges may have changed


def _try_fused_zero(optimizer: "Optimizer") -> Any:
    """The in-kernel NVLink path of the ZeRO step, if symmetric memory is available for the group.

    The decision is taken by the data-parallel group as a whole: a rank on which the set-up failed must not fall
    back to library collectives while its peers wait at flag barriers, so the ranks exchange a success flag and
    use the peer-memory kernels only if every one of them has them."""
    t = optimizer.topology
    fused = None
    error = ""
    try:
        from ...parallel.fused_zero import FusedZero

        fused = FusedZero.create(optimizer)
    except Exception as e:  # pragma: no cover - depends on the machine
        error = f"{type(e).__name__}: {e}"
    ok = torch.tensor([1.0 if fused is not None else 0.0], device=t.device)
    if t.is_distributed_initialized:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=t.data_parallel_group)
    if ok.item() < 1.0:
        if fused is not None:
            logger.warning("fused NVLink ZeRO path available here but not on every data-parallel rank; using NCCL")
        elif error:
            logger.warning(f"fused NVLink ZeRO path unavailable ({error}); using NCCL collectives")
        return None  # the buffers of groups that already moved into symmetric memory stay valid as plain tensors
    logger.info("ZeRO data-parallel exchange: peer-memory kernels over NVLink "
                f"(multicast stores: {'yes' if fused.use_multicast else 'no'})")
    return fused
