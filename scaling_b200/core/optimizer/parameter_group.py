"""One optimizer parameter group: flat low-precision parameters and gradients, fp32 master state.

At ``initialize`` the group's parameters are packed into ONE flat buffer on the device (each start
aligned to 128 bytes so that every weight remains a valid TMA source), ``param.data`` is re-pointed
into it and ``param.grad`` becomes a permanent view of a second flat buffer, so gradients of all
micro batches accumulate in place and the data-parallel reduction is a single collective over
contiguous memory.  The fp32 master weights and the Adam moments exist either for the whole buffer
or, with ZeRO stage 1, only for this data-parallel rank's equal share of it
(partition ``d`` = elements ``[d * n, (d + 1) * n)`` of the padded buffer, as in
src/scaling/core/optimizer/parameter_group.py:28-80,143-238 - but built on the device, without the
reference's round trip through host memory).

Order inside the buffer: tensor-parallel sharded parameters, then replicated ones, then replicated
ones whose gradients are partial per rank (sequence-parallel norms, replicated KV projections).  The
gradient norm then needs at most two range reductions and the extra tensor-parallel gradient
reduction is one collective over one slice.
"""

from __future__ import annotations

from typing import Any, List, Optional, Tuple

import torch

from ...parallel.topology import Topology
from ..nn.parameter_meta import CoreParameterMeta
from .learning_rate_scheduler import LearningRateScheduler
from .optimizer_config import OptimizerParamGroupConfig

ALIGN_ELEMENTS = 64


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


def needs_model_parallel_grad_reduce(name: str, p: torch.Tensor, topology: Topology) -> bool:
    if topology.config.model_parallel_size == 1:
        return False
    # set by the modules whose replicated parameters receive partial gradients per rank: norms under
    # sequence parallelism, biases added on one rank only, KV projections replicated for MQA
    return bool(getattr(p, "reduce_grad_over_model_parallel", False))


class OptimizerParamGroup:
    def __init__(self, named_parameters_with_meta: List[Tuple[str, torch.Tensor, CoreParameterMeta]],
                 config: OptimizerParamGroupConfig):
        self.config = config
        self.learning_rate_scheduler = LearningRateScheduler(config.learning_rate_scheduler)
        self.parameter_names: List[str] = []
        self.parameter_metas: List[CoreParameterMeta] = []
        self.parameters_original: List[torch.Tensor] = []
        for n, p, m in named_parameters_with_meta:
            self.parameter_names.append(n)
            self.parameters_original.append(p)
            self.parameter_metas.append(m)
        self.initialized = False
        self.zero = False
        self.current_lr = 0.0

    # ------------------------------------------------------------------ construction
    def initialize(self, topology: Topology, zero: bool) -> None:
        self.zero = zero
        dp = topology.config.data_parallel_size
        self.dp, self.dp_rank = dp, topology.data_parallel_rank
        params = self.parameters_original
        if params:
            dtypes = {p.dtype for p in params}
            assert len(dtypes) == 1, f"all parameters of an optimizer group must share one dtype, got {dtypes}"
            self.dtype = params[0].dtype
            self.device = params[0].device
        else:  # a stage may hold no parameter of a group; keep an empty, well-formed group
            self.dtype = torch.float32
            self.device = topology.device

        def rank_of(i: int) -> int:
            if needs_model_parallel_grad_reduce(self.parameter_names[i], params[i], topology):
                return 2
            return 0 if self.parameter_metas[i].is_model_parallel else 1

        # classes are taken before the lists are permuted (rank_of indexes them)
        class_of = [rank_of(i) for i in range(len(params))]
        order = sorted(range(len(params)), key=lambda i: (class_of[i], i))
        classes = [class_of[i] for i in order]
        self.parameter_names = [self.parameter_names[i] for i in order]
        self.parameter_metas = [self.parameter_metas[i] for i in order]
        self.parameters_original = params = [params[i] for i in order]

        self.offsets: list[int] = []
        cursor = 0
        seg_end = [0, 0, 0]
        for p, cls in zip(params, classes):
            self.offsets.append(cursor)
            cursor = _align(cursor + p.numel(), ALIGN_ELEMENTS)
            seg_end[cls] = cursor
        seg_end[1] = max(seg_end[1], seg_end[0])
        seg_end[2] = max(seg_end[2], seg_end[1])
        self.segment_ends = seg_end  # [sharded | replicated | replicated with partial grads)
        self.numel = cursor
        self.padded_numel = max(_align(cursor, 2 * dp * ALIGN_ELEMENTS), 2 * dp * ALIGN_ELEMENTS)
        self.partition_numel = self.padded_numel // dp

        self.step_ranges: list[tuple[int, int, int]] = [(0, self.padded_numel, 0)]  # (start, end, born): see below
        self.flat_param = torch.zeros(self.padded_numel, dtype=self.dtype, device=self.device)
        self.flat_grad = torch.zeros(self.padded_numel, dtype=self.dtype, device=self.device)
        with torch.no_grad():
            for p, off in zip(params, self.offsets):
                view = self.flat_param[off:off + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.grad = self.flat_grad[off:off + p.numel()].view(p.shape)
                # backward kernels may add into this persistent buffer from their epilogue
                p.fused_grad_accumulation = True  # type: ignore[attr-defined]

        lo, hi = self.owned_range
        if self.dtype == torch.float32:
            self.master = self.flat_param[lo:hi]  # fp32 training: the parameters are their own master copy
        else:
            self.master = self.flat_param[lo:hi].float()
        self.exp_avg = torch.zeros(hi - lo, dtype=torch.float32, device=self.device)
        self.exp_avg_sq = torch.zeros(hi - lo, dtype=torch.float32, device=self.device)
        # reduced gradient of the owned range (ZeRO: output of the reduce-scatter)
        self.reduced_grad: Optional[torch.Tensor] = (
            torch.zeros(hi - lo, dtype=self.dtype, device=self.device) if (zero and dp > 1) else None
        )
        wd = self.config.weight_decay
        if self.config.independent_weight_decay:
            wd = wd / self.config.learning_rate_scheduler.learning_rate
        self.weight_decay = wd
        self.initialized = True

    def rehome(self, flat_param: torch.Tensor, flat_grad: torch.Tensor) -> None:
        """Move the flat parameter and gradient buffers into caller-provided storage of the same size and dtype
        (e.g. symmetric memory that peers can address); parameters and their ``.grad`` become views of it."""
        assert self.initialized
        assert flat_param.shape == self.flat_param.shape and flat_param.dtype == self.flat_param.dtype
        assert flat_grad.shape == self.flat_grad.shape and flat_grad.dtype == self.flat_grad.dtype
        with torch.no_grad():
            flat_param.copy_(self.flat_param)
            flat_grad.copy_(self.flat_grad)
            for p, off in zip(self.parameters_original, self.offsets):
                p.data = flat_param[off:off + p.numel()].view(p.shape)
                p.grad = flat_grad[off:off + p.numel()].view(p.shape)
        self.flat_param, self.flat_grad = flat_param, flat_grad
        if self.dtype == torch.float32:
            lo, hi = self.owned_range
            self.master = self.flat_param[lo:hi]

    @property
    def owned_range(self) -> tuple[int, int]:
        """Element range of the flat buffer whose optimizer state lives on this rank."""
        if self.zero:
            return self.dp_rank * self.partition_numel, (self.dp_rank + 1) * self.partition_numel
        return 0, self.padded_numel

    def norm_ranges(self, topology: Topology) -> list[tuple[int, int]]:
        """Ranges (relative to the owned range) that count towards the global gradient norm on this rank:
        sharded parameters everywhere, replicated ones only on tensor-parallel rank 0."""
        lo, hi = self.owned_range
        end = self.padded_numel if topology.model_parallel_rank == 0 else self.segment_ends[0]
        a, b = max(lo, 0), min(hi, end)
        if b <= a:
            return []
        # copies of a weight tied to an earlier pipeline stage are not counted again (the reference counts every
        # copy, which makes gradient clipping depend on the layout)
        ranges = [(a, b)]
        for p, (s0, s1) in zip(self.parameters_original, self.param_slices()):
            if not getattr(p, "tied_copy_of_earlier_stage", False):
                continue
            cut: list[tuple[int, int]] = []
            for r0, r1 in ranges:
                if s1 <= r0 or s0 >= r1:
                    cut.append((r0, r1))
                    continue
                if r0 < s0:
                    cut.append((r0, s0))
                if s1 < r1:
                    cut.append((s1, r1))
            ranges = cut
        return [(r0 - lo, r1 - lo) for r0, r1 in ranges if r1 > r0]

    # ------------------------------------------------------------------ step helpers
    def set_learning_rate(self, step_index: int) -> float:
        self.current_lr = self.learning_rate_scheduler.get_lr(step_index)
        return self.current_lr

    def get_learning_rate(self) -> float:
        return self.current_lr

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.flat_grad.zero_()

    def refresh_optimized_params(self, topology: Optional[Topology] = None) -> None:
        """Master copy <- current low-precision parameters (after a model-only checkpoint load)."""
        lo, hi = self.owned_range
        if self.dtype != torch.float32:
            self.master.copy_(self.flat_param[lo:hi])

    # ------------------------------------------------------------------ age of the Adam state
    def set_parameter_steps(self, born: list[int]) -> None:
        """``born[i]``: how many optimizer updates had been applied when parameter ``i``'s moments started from zero.
        Neighbouring parameters of equal age are merged into one range (one AdamW launch each)."""
        ranges: list[tuple[int, int, int]] = []
        slices = self.param_slices()
        for i, ((a, _), age) in enumerate(zip(slices, born)):
            end = slices[i + 1][0] if i + 1 < len(slices) else self.padded_numel
            start = 0 if i == 0 else a
            if ranges and ranges[-1][2] == age:
                ranges[-1] = (ranges[-1][0], end, age)
            else:
                ranges.append((start, end, age))
        self.step_ranges = ranges or [(0, self.padded_numel, 0)]

    def born_at(self, offset: int) -> int:
        for a, b, age in self.step_ranges:
            if a <= offset < b:
                return age
        return 0

    # ------------------------------------------------------------------ views for checkpoints
    def param_slices(self) -> list[tuple[int, int]]:
        return [(off, off + p.numel()) for p, off in zip(self.parameters_original, self.offsets)]

    def state_dict(self) -> dict[str, Any]:
        return {
            "parameter_names": list(self.parameter_names),
            "parameter_metas": [m.state_dict() for m in self.parameter_metas],
            "offsets": list(self.offsets),
            "owned_range": self.owned_range,
            "padded_numel": self.padded_numel,
            "master": self.master.detach().clone().cpu(),
            "exp_avg": self.exp_avg.detach().clone().cpu(),
            "exp_avg_sq": self.exp_avg_sq.detach().clone().cpu(),
            "zero": self.zero,
            "step_ranges": [list(r) for r in self.step_ranges],
        }

    def load_state_dict(self, state: dict[str, Any]) -> None:
        assert tuple(state["owned_range"]) == tuple(self.owned_range) and state["padded_numel"] == self.padded_numel, (
            "static optimizer state was written with a different layout"
        )
        self.master.copy_(state["master"])
        self.exp_avg.copy_(state["exp_avg"])
        self.exp_avg_sq.copy_(state["exp_avg_sq"])
        self.step_ranges = [tuple(r) for r in state.get("step_ranges", [(0, self.padded_numel, 0)])]
        self.write_back_params()

    def write_back_params(self) -> None:
        lo, hi = self.owned_range
        if self.dtype != torch.float32:
            self.flat_param[lo:hi].copy_(self.master)
