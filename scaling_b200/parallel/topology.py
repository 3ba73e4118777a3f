"""3-D rank grid (pipe x data x model), process groups and device binding.

Ranks are laid out as ``rank = (pipe * dp + data) * mp + model`` so that tensor-parallel peers are
adjacent (same NVSwitch domain) - the layout of the reference
(src/scaling/core/topology/topology.py:45-55).  Every rank creates every group in the same order.
Differences to the reference, on purpose: the backend and device are configurable (``gloo``/``cpu``
make all host-side logic testable without GPUs), and peer-addressable symmetric buffers for the
fused compute+collective kernels are obtained per group through ``symmetric`` on demand.
"""

from __future__ import annotations

import datetime
import os
from typing import Any, Optional, TypedDict

import numpy as np
import torch
import torch.distributed as dist

from .rng_tracker import CudaRNGStateTracker, KernelDropoutState, RngTrackerState
from .topology_config import TopologyConfig


# Point-to-point groups between pipeline stages use at most this many CTAs per NCCL kernel; up to four such kernels
# can be active at once on a middle stage (receive and send, in each direction).
PIPE_P2P_MAX_CTAS = 2
PIPE_P2P_RESERVED_SMS = 4 * PIPE_P2P_MAX_CTAS


def _destroy_process_group_quietly() -> None:
    try:
        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
    except Exception:  # noqa: BLE001 - the process is exiting anyway
        pass


class TopologyState(TypedDict):
    model_parallel_constant_rng: RngTrackerState


class Topology:
    def __init__(self, config: TopologyConfig):
        self.config = config
        self.world_size = config.world_size
        self.model_parallel_size = config.model_parallel_size
        self.pipe_parallel_size = config.pipe_parallel_size
        self.data_parallel_size = config.data_parallel_size
        self.global_batch_size = config.global_batch_size
        self.micro_batch_size = config.micro_batch_size
        self.gradient_accumulation_steps = config.gradient_accumulation_steps
        self.pipe_partition_method = config.pipe_partition_method
        self.pipe_partition_overwrite = config.pipe_partition_overwrite
        self.activation_checkpointing_type = config.activation_checkpointing_type
        self.sequence_parallel = config.sequence_parallel

        self._grid = np.arange(self.world_size).reshape(
            self.pipe_parallel_size, self.data_parallel_size, self.model_parallel_size
        )
        self._pipe_group = self._data_group = self._model_group = None
        self._rng: Optional[CudaRNGStateTracker] = None
        self._kernel_rng: Optional[KernelDropoutState] = None
        self.is_distributed_initialized = False
        self._device: Optional[torch.device] = None

        if config.global_rank is not None:
            pp, dp, mp = (int(v[0]) for v in np.where(self._grid == config.global_rank))
            self._pp, self._dp, self._mp = pp, dp, mp
        else:
            self._pp = self._dp = self._mp = None  # type: ignore[assignment]

    # ------------------------------------------------------------------ device / backend
    @property
    def device_type(self) -> str:
        if self.config.device is not None:
            return self.config.device
        return "cuda" if torch.cuda.is_available() else "cpu"

    @property
    def backend(self) -> str:
        if self.config.backend is not None:
            return self.config.backend
        return "nccl" if self.device_type == "cuda" else "gloo"

    @property
    def device(self) -> torch.device:
        if self._device is None:
            if self.device_type == "cuda":
                slot = self.config.local_slot if self.config.local_slot is not None else 0
                self._device = torch.device("cuda", slot)
            else:
                self._device = torch.device("cpu")
        return self._device

    def initialize_device(self) -> None:
        if self.device_type == "cuda":
            assert self.config.local_slot is not None, "local_slot must be set to bind a CUDA device"
            torch.cuda.set_device(self.config.local_slot)

    # ------------------------------------------------------------------ distributed init
    def initialize_distributed(
        self,
        master_addr: Optional[str] = None,
        master_port: Optional[str] = None,
        torch_distributed_timeout_minutes: int = 20,
        seed: int = 42,
    ) -> None:
        assert self.config.global_rank is not None, "global_rank is required to initialize torch.distributed"
        self.initialize_device()
        # same seed on all model-parallel ranks of one (pipe, data) cell
        cell_seed = seed + self.get_global_rank(model_parallel_rank=0)
        self._rng = CudaRNGStateTracker(cell_seed, device=self.device)
        self._kernel_rng = KernelDropoutState(cell_seed, self.device)
        if not dist.is_initialized():
            addr = master_addr or os.environ.get("MASTER_ADDR", "127.0.0.1")
            port = master_port or os.environ.get("MASTER_PORT", "29500")
            kwargs: dict[str, Any] = {}
            if self.device_type == "cuda":
                kwargs["device_id"] = self.device
            dist.init_process_group(
                backend=self.backend,
                init_method=f"tcp://{addr}:{port}",
                world_size=self.world_size,
                rank=self.config.global_rank,
                timeout=datetime.timedelta(minutes=torch_distributed_timeout_minutes),
                **kwargs,
            )
            if self.backend == "gloo":
                # CPU ranks: tear the group down at interpreter exit.  A gloo group that is still alive when the
                # process ends can abort it ("terminate called without an active exception") after the work is done.
                # Not for NCCL: its teardown waits for the peers, and a rank that exits after a failure must not.
                import atexit

                atexit.register(_destroy_process_group_quietly)
        for ranks in self.all_pipe_parallel_groups:
            g = dist.new_group(ranks)
            if self.config.global_rank in ranks:
                self._pipe_group = g
        if self.pipe_parallel_size > 1:
            # Point-to-point traffic between stages: one group per direction (activations towards the last stage,
            # gradients towards the first).  Each group has its own communicators and streams, so a receive that is
            # posted ahead of time in one direction never queues in front of a send in the other.  On NCCL the
            # groups are limited to a few CTAs per kernel: a copy between two GPUs needs no more, and kernels that
            # wait for their tensor-parallel peers leave that many SMs free (PIPE_P2P_RESERVED_SMS).
            for ranks in self.all_pipe_parallel_groups:
                for direction in ("down", "up"):
                    g = dist.new_group(ranks, pg_options=self._p2p_group_options())
                    if self.config.global_rank in ranks:
                        setattr(self, f"_pipe_{direction}_group", g)
        for ranks in self.all_data_parallel_groups:
            g = dist.new_group(ranks)
            if self.config.global_rank in ranks:
                self._data_group = g
        for ranks in self.all_model_parallel_groups:
            g = dist.new_group(ranks)
            if self.config.global_rank in ranks:
                self._model_group = g
        self.is_distributed_initialized = True

    def _p2p_group_options(self) -> Any:
        if self.backend != "nccl":
            return None
        try:
            opts = dist.ProcessGroupNCCL.Options()
            opts.config.max_ctas = PIPE_P2P_MAX_CTAS
            opts.config.min_ctas = 1
            return opts
        except Exception:  # pragma: no cover - older builds without per-group NCCL configuration
            return None

    @property
    def pipe_down_group(self) -> Any:
        """Group that carries activations from a stage to the next (None without pipeline parallelism)."""
        return getattr(self, "_pipe_down_group", None)

    @property
    def pipe_up_group(self) -> Any:
        """Group that carries gradients (and the loss record) from a stage to an earlier one."""
        return getattr(self, "_pipe_up_group", None)

    @property
    def reserved_sms(self) -> int:
        """SMs that kernels waiting on their tensor-parallel peers must leave free on this layout: with pipeline
        stages, send / receive kernels of the two point-to-point groups run beside the compute stream, and a kernel
        whose CTAs wait for CTAs of another GPU must be completely resident however many of those are active."""
        return PIPE_P2P_RESERVED_SMS if self.pipe_parallel_size > 1 else 0

    # ------------------------------------------------------------------ rng
    @property
    def has_model_parallel_constant_rng(self) -> bool:
        return self._rng is not None

    @property
    def model_parallel_constant_rng(self):
        assert self._rng is not None, "topology is not initialized"
        return self._rng.fork

    @property
    def kernel_rng(self) -> KernelDropoutState:
        """Counter-based random stream of the dropout kernels; the same on all tensor-parallel ranks of a replica."""
        if self._kernel_rng is None:  # single process without torch.distributed
            self._kernel_rng = KernelDropoutState(42 + (self.config.global_rank or 0), self.device)
        return self._kernel_rng

    def state_dict(self) -> Optional[TopologyState]:
        if self._rng is None:
            return None
        return {"model_parallel_constant_rng": self._rng.state_dict(),  # type: ignore[typeddict-unknown-key]
                "kernel_rng": self.kernel_rng.state_dict()}

    def load_state_dict(self, state_dict: Optional[dict[str, Any]]) -> None:
        if state_dict is None or self._rng is None:
            return
        self._rng.load_state_dict(state_dict["model_parallel_constant_rng"])
        if "kernel_rng" in state_dict:
            self.kernel_rng.load_state_dict(state_dict["kernel_rng"])

    # ------------------------------------------------------------------ coordinates
    def _need_rank(self) -> None:
        assert self.config.global_rank is not None, "global_rank is not set"

    @property
    def pipe_parallel_rank(self) -> int:
        self._need_rank()
        return self._pp

    @property
    def data_parallel_rank(self) -> int:
        self._need_rank()
        return self._dp

    @property
    def model_parallel_rank(self) -> int:
        self._need_rank()
        return self._mp

    @property
    def previous_pipe_parallel_rank(self) -> Optional[int]:
        return None if self.pipe_parallel_rank == 0 else self.pipe_parallel_rank - 1

    @property
    def next_pipe_parallel_rank(self) -> Optional[int]:
        return None if self.pipe_parallel_rank == self.pipe_parallel_size - 1 else self.pipe_parallel_rank + 1

    @property
    def is_first_pipe_parallel_rank(self) -> bool:
        return self.pipe_parallel_rank == 0

    @property
    def is_last_pipe_parallel_rank(self) -> bool:
        return self.pipe_parallel_rank == self.pipe_parallel_size - 1

    @property
    def is_first_model_parallel_rank(self) -> bool:
        return self.model_parallel_rank == 0

    @property
    def is_io_rank(self) -> bool:
        """Ranks that load data: first or last pipeline stage, model-parallel rank 0."""
        return (self.is_first_pipe_parallel_rank or self.is_last_pipe_parallel_rank) and self.is_first_model_parallel_rank

    # ranks that share this rank's other two coordinates
    @property
    def pipe_parallel_ranks(self) -> list[int]:
        self._need_rank()
        return [int(r) for r in self._grid[:, self._dp, self._mp]]

    @property
    def data_parallel_ranks(self) -> list[int]:
        self._need_rank()
        return [int(r) for r in self._grid[self._pp, :, self._mp]]

    @property
    def model_parallel_ranks(self) -> list[int]:
        self._need_rank()
        return [int(r) for r in self._grid[self._pp, self._dp, :]]

    @property
    def pipe_parallel_group(self):
        assert self._pipe_group is not None, "distributed is not initialized"
        return self._pipe_group

    @property
    def data_parallel_group(self):
        assert self._data_group is not None, "distributed is not initialized"
        return self._data_group

    @property
    def model_parallel_group(self):
        assert self._model_group is not None, "distributed is not initialized"
        return self._model_group

    @property
    def all_pipe_parallel_groups(self) -> list[list[int]]:
        return [
            [int(r) for r in self._grid[:, d, m]]
            for d in range(self.data_parallel_size)
            for m in range(self.model_parallel_size)
        ]

    @property
    def all_data_parallel_groups(self) -> list[list[int]]:
        return [
            [int(r) for r in self._grid[p, :, m]]
            for p in range(self.pipe_parallel_size)
            for m in range(self.model_parallel_size)
        ]

    @property
    def all_model_parallel_groups(self) -> list[list[int]]:
        return [
            [int(r) for r in self._grid[p, d, :]]
            for p in range(self.pipe_parallel_size)
            for d in range(self.data_parallel_size)
        ]

    def get_global_rank(
        self,
        pipe_parallel_rank: Optional[int] = None,
        data_parallel_rank: Optional[int] = None,
        model_parallel_rank: Optional[int] = None,
    ) -> int:
        """Global rank at the given coordinates; omitted coordinates default to this rank's own."""
        p = self.pipe_parallel_rank if pipe_parallel_rank is None else pipe_parallel_rank
        d = self.data_parallel_rank if data_parallel_rank is None else data_parallel_rank
        m = self.model_parallel_rank if model_parallel_rank is None else model_parallel_rank
        return int(self._grid[p, d, m])

    def get_global_rank_group(
        self,
        pipe_parallel_rank: Optional[int] = None,
        data_parallel_rank: Optional[int] = None,
        model_parallel_rank: Optional[int] = None,
        flatten: bool = True,
    ) -> list:
        """All global ranks matching the given coordinates (None = wildcard); ``flatten=False`` keeps the
        ``[pipe][data][model]`` nesting."""
        sel = self._grid[
            slice(None) if pipe_parallel_rank is None else [pipe_parallel_rank],
            :,
            :,
        ]
        sel = sel[:, slice(None) if data_parallel_rank is None else [data_parallel_rank], :]
        sel = sel[:, :, slice(None) if model_parallel_rank is None else [model_parallel_rank]]
        return [int(r) for r in sel.flatten()] if flatten else sel.tolist()
