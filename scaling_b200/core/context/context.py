"""Run-time state of one training or inference process.

Holds the immutable config, the topology and the progress counters; seeds all generators with
``seed + global_rank``; writes one ``context_global_rank_{r}.pt`` per rank plus ``config.yml`` from
rank 0 (layout of src/scaling/core/context/context.py:91-161).  When a checkpoint is resumed with
more ranks than it was written with, the counters are synchronised with an all-reduce(MAX).
"""

from __future__ import annotations

import random
from pathlib import Path
from typing import Any, Generic, Optional, TypedDict, TypeVar

import numpy as np
import torch
import torch.distributed as dist

from ...parallel.topology import Topology
from ..config import BaseConfig


class ContextState(TypedDict, total=False):
    iterations: int
    consumed_samples: int
    consumed_samples_evaluation: int
    random_rng_state: Any
    np_rng_state: Any
    torch_rng_state: Any
    torch_cuda_rng_state: Any
    topology: Any


class BaseContext:
    def __init__(self, config: BaseConfig, topology: Topology) -> None:
        self.config = config
        self.topology = topology
        self.iterations = 0
        self.consumed_samples = 0
        self.consumed_samples_evaluation = 0

    def initialize(self, master_addr: str, master_port: str, torch_distributed_timeout_minutes: int = 20,
                   seed: int = 42, distributed: bool = True) -> None:
        if self.topology is not None:
            if distributed:
                self.topology.initialize_distributed(
                    seed=seed, master_addr=master_addr, master_port=str(master_port),
                    torch_distributed_timeout_minutes=torch_distributed_timeout_minutes,
                )
            else:
                self.topology.initialize_device()
            assert self.topology.config.global_rank is not None
            seed = seed + self.topology.config.global_rank
        random.seed(seed)
        np.random.seed(seed)
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed(seed)

    def step(self) -> None:
        self.iterations += 1
        self.consumed_samples += self.topology.config.global_batch_size

    def _on_cuda(self) -> bool:
        return self.topology is not None and self.topology.device_type == "cuda" and torch.cuda.is_available()

    def state_dict(self) -> ContextState:
        return {
            "iterations": self.iterations,
            "consumed_samples": self.consumed_samples,
            "consumed_samples_evaluation": self.consumed_samples_evaluation,
            "random_rng_state": random.getstate(),
            "np_rng_state": np.random.get_state(),
            "torch_rng_state": torch.get_rng_state(),
            "torch_cuda_rng_state": torch.cuda.get_rng_state() if self._on_cuda() else None,
            "topology": self.topology.state_dict(),
        }

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self.iterations = state_dict["iterations"]
        self.consumed_samples = state_dict["consumed_samples"]
        self.consumed_samples_evaluation = state_dict.get("consumed_samples_evaluation", 0)
        random.setstate(state_dict["random_rng_state"])
        np.random.set_state(state_dict["np_rng_state"])
        torch.set_rng_state(state_dict["torch_rng_state"])
        if state_dict.get("torch_cuda_rng_state") is not None and self._on_cuda():
            torch.cuda.set_rng_state(state_dict["torch_cuda_rng_state"])
        self.topology.load_state_dict(state_dict.get("topology"))

    def save_checkpoint(self, dir: Path | str) -> None:
        dir = Path(dir)
        dir.mkdir(parents=True, exist_ok=True)
        rank = self.topology.config.global_rank
        if rank == 0:
            self.config.save(dir / "config.yml")
        torch.save(self.state_dict(), str(dir / f"context_global_rank_{rank}.pt"))

    def load_checkpoint(self, dir: Path | str) -> None:
        dir = Path(dir)
        f = dir / f"context_global_rank_{self.topology.config.global_rank}.pt"
        if f.is_file():
            # the file pickles python / numpy generator states, hence weights_only=False
            self.load_state_dict(torch.load(str(f), weights_only=False))
        if self.topology.is_distributed_initialized:
            t = torch.tensor(
                [self.iterations, self.consumed_samples, self.consumed_samples_evaluation],
                dtype=torch.int64, device=self.topology.device,
            )
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            self.iterations, self.consumed_samples, self.consumed_samples_evaluation = (int(v) for v in t.tolist())


BaseContextGeneric = TypeVar("BaseContextGeneric", bound=BaseContext)


class DeterminedBaseContext(BaseContext):
    """Context that additionally carries a Determined core context (optional dependency)."""

    def __init__(self, config: BaseConfig, topology: Topology) -> None:
        super().__init__(config=config, topology=topology)
        self.determined_context: Optional[Any] = None
        self.determined_profiler: Optional[Any] = None
        self._use_determined = False

    def initialize_with_determined(self, master_addr: str, master_port: str, determined_context: Any,
                                   determined_profiler: Optional[Any], torch_distributed_timeout_minutes: int = 20,
                                   seed: int = 42, distributed: bool = True) -> None:
        super().initialize(master_addr, master_port, torch_distributed_timeout_minutes, seed, distributed)
        self.determined_context = determined_context
        self.determined_profiler = determined_profiler
        self._use_determined = True
