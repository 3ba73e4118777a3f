"""Random-number streams that are identical on all tensor-parallel ranks of a replica.

Dropout on activations that are replicated inside a TP group must draw the same mask on every rank
of the group.  The tracker keeps a second generator state seeded per (pipe, data) cell; ``fork()``
swaps it in for the duration of a block and stores the advanced state afterwards
(reference: src/scaling/core/topology/rng_tracker.py:59-95).  On CPU ranks the same mechanism runs
on the default CPU generator so that the logic is testable without a GPU.
"""

from __future__ import annotations

import contextlib
from typing import Iterator, TypedDict

import torch


class RngTrackerState(TypedDict):
    seed: int
    state: torch.Tensor


class _Backend:
    def __init__(self, device: torch.device):
        self.cuda = device.type == "cuda"
        self.index = device.index if device.index is not None else (torch.cuda.current_device() if self.cuda else 0)

    def get(self) -> torch.Tensor:
        if self.cuda:
            return torch.cuda.default_generators[self.index].get_state()
        return torch.get_rng_state()

    def set(self, state: torch.Tensor) -> None:
        # set_state on the generator does not clone the tensor, unlike torch.cuda.set_rng_state
        if self.cuda:
            torch.cuda.default_generators[self.index].set_state(state)
        else:
            torch.set_rng_state(state)

    def seed(self, seed: int) -> None:
        if self.cuda:
            torch.cuda.default_generators[self.index].manual_seed(seed)
        else:
            torch.manual_seed(seed)


class CudaRNGStateTracker:
    def __init__(self, seed: int, device: torch.device | None = None):
        device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self._be = _Backend(device)
        self.seed = seed
        outer = self._be.get()
        self._be.seed(seed)
        self.state = self._be.get()
        self._be.set(outer)

    def state_dict(self) -> RngTrackerState:
        return {"seed": self.seed, "state": self.state.clone().detach()}

    def load_state_dict(self, state_dict: RngTrackerState) -> None:
        self.seed = state_dict["seed"]
        self.state = state_dict["state"].cpu().to(torch.uint8)

    @contextlib.contextmanager
    def fork(self) -> Iterator[None]:
        outer = self._be.get()
        self._be.set(self.state)
        try:
            yield
        finally:
            self.state = self._be.get()
            self._be.set(outer)


class KernelDropoutState:
    """Random stream of the dropout kernels (residual dropout, attention dropout inside the flash kernel).

    The kernels are counter based: a mask is a function of ``(seed, step, call, element)``.  ``seed`` and ``step`` live
    in a device tensor that the kernels read (so a captured CUDA graph draws fresh masks on every replay once
    ``begin_step`` has advanced the step), ``call`` numbers the dropout sites in the order they run inside a step and is
    passed to each launch.  The seed is the same on all tensor-parallel ranks of a replica, like the generator of
    ``CudaRNGStateTracker``; backward passes and recomputed forward passes rebuild their mask from the same triple
    (activation checkpointing saves and restores ``call_index``).
    """

    def __init__(self, seed: int, device: torch.device):
        self.seed = int(seed)
        self.device = device
        self.step = 0
        self.call_index = 0
        self._device_state: torch.Tensor | None = None
        self._host_state: torch.Tensor | None = None

    def _upload(self) -> None:
        if self._device_state is None:
            self._host_state = torch.zeros(2, dtype=torch.int64, pin_memory=self.device.type == "cuda")
            self._device_state = torch.zeros(2, dtype=torch.int64, device=self.device)
        assert self._host_state is not None
        self._host_state[0] = self.seed
        self._host_state[1] = self.step
        self._device_state.copy_(self._host_state, non_blocking=True)

    def tensor(self) -> torch.Tensor:
        """Device int64[2] ``{seed, step}``."""
        if self._device_state is None:
            self._upload()
        assert self._device_state is not None
        return self._device_state

    def begin_step(self) -> None:
        """Start of a training step: new masks everywhere, call numbering starts over."""
        self.step += 1
        self.call_index = 0
        self._upload()

    def next_call(self) -> int:
        c = self.call_index
        self.call_index += 1
        return c

    def state_dict(self) -> dict[str, int]:
        return {"seed": self.seed, "step": self.step}

    def load_state_dict(self, state: dict[str, int]) -> None:
        self.seed, self.step = int(state["seed"]), int(state["step"])
        self.call_index = 0
        if self._device_state is not None:
            self._upload()
