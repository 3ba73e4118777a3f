"""Activation checkpointing that also rewinds the tensor-parallel-constant RNG stream.

The forward of a checkpointed block runs without building a graph and keeps only the block's
inputs together with the generator states (CPU, current CUDA device, the topology's
model-parallel-constant tracker, and the call counter of the counter-based dropout kernels).  During backward the states are restored, the block is run
again with autograd enabled, and gradients flow through the recomputed graph.  Dropout therefore
draws identical masks in the first and the recomputed pass, on every tensor-parallel rank.
Same guarantee as the reference's fork of torch's non-reentrant checkpoint
(src/scaling/core/nn/parallel_module/activation_checkpointing.py:72-190); this implementation is
a custom autograd function over flat tuples, which is the form the pipeline engine already uses.
"""

from __future__ import annotations

from typing import Any, Callable, Optional, Sequence

import torch

from ....parallel.topology import Topology


def _capturing() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_initialized() and torch.cuda.is_current_stream_capturing()


def _capture_rng(topology: Optional[Topology]) -> dict[str, Any]:
    # the dropout kernels number their calls inside a step on the host: the recomputed pass starts from the number
    # the first pass started from (a plain integer, also while a CUDA graph is being captured)
    calls = {"kernel_rng_call": topology.kernel_rng.call_index} if topology is not None else {}
    if _capturing():
        return calls  # generator states cannot be read under capture; a captured step uses the dropout kernels only
    state: dict[str, Any] = dict(calls, cpu=torch.get_rng_state())
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        state["cuda"] = torch.cuda.get_rng_state()
    if topology is not None and topology.has_model_parallel_constant_rng:
        state["topology"] = topology.state_dict()
    return state


def _restore_rng(state: dict[str, Any], topology: Optional[Topology]) -> None:
    if "kernel_rng_call" in state and topology is not None:
        topology.kernel_rng.call_index = state["kernel_rng_call"]
    if "cpu" not in state:
        return
    torch.set_rng_state(state["cpu"])
    if "cuda" in state:
        torch.cuda.set_rng_state(state["cuda"])
    if "topology" in state and topology is not None:
        topology.load_state_dict(state["topology"])


class _Checkpoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run: Callable, topology: Optional[Topology], anchor: torch.Tensor, *args: Any):  # type: ignore[override]
        ctx.run = run
        ctx.topology = topology
        ctx.rng = _capture_rng(topology)
        ctx.is_tensor = [isinstance(a, torch.Tensor) for a in args]
        ctx.others = [None if t else a for a, t in zip(args, ctx.is_tensor)]
        ctx.save_for_backward(*[a for a in args if isinstance(a, torch.Tensor)])
        ctx.req = [isinstance(a, torch.Tensor) and a.requires_grad for a in args]
        with torch.no_grad():
            out = run(*args)
        ctx.out_is_tuple = isinstance(out, tuple)
        outs = out if ctx.out_is_tuple else (out,)
        ctx.out_tensor = [isinstance(o, torch.Tensor) for o in outs]
        # non-differentiable outputs (integer tensors, python objects) are passed through untouched
        nondiff = [o for o in outs if isinstance(o, torch.Tensor) and not o.is_floating_point()]
        if nondiff:
            ctx.mark_non_differentiable(*nondiff)
        return out

    @staticmethod
    def backward(ctx, *grads: Any):  # type: ignore[override]
        saved = list(ctx.saved_tensors)
        args = []
        for is_t, other, req in zip(ctx.is_tensor, ctx.others, ctx.req):
            if is_t:
                t = saved.pop(0).detach()
                t.requires_grad_(req)
                args.append(t)
            else:
                args.append(other)
        outer = _capture_rng(ctx.topology)
        _restore_rng(ctx.rng, ctx.topology)
        try:
            with torch.enable_grad():
                out = ctx.run(*args)
        finally:
            _restore_rng(outer, ctx.topology)
        outs = out if isinstance(out, tuple) else (out,)
        pairs = [
            (o, g) for o, g in zip(outs, grads)
            if isinstance(o, torch.Tensor) and o.requires_grad and g is not None
        ]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        in_grads = [a.grad if isinstance(a, torch.Tensor) and a.requires_grad else None for a in args]
        return (None, None, None, *in_grads)


def checkpoint(function: Callable, topology: Optional[Topology], *args: Any) -> Any:
    """Run ``function(*args)`` now, recompute it in backward instead of storing its activations."""
    # the anchor makes the output part of the graph even if no input requires grad (first stage: token ids)
    anchor = torch.zeros((), requires_grad=True, device=_first_device(args))
    return _Checkpoint.apply(function, topology, anchor, *args)


def _first_device(args: Sequence[Any]) -> torch.device:
    for a in args:
        if isinstance(a, torch.Tensor):
            return a.device
    return torch.device("cpu")
