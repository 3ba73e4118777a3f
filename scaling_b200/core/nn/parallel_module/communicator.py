"""Point-to-point exchange of arbitrary pytrees between neighbouring pipeline stages.

Wire protocol (equivalent in effect to src/scaling/core/nn/parallel_module/communicator.py:286-482):
the payload is flattened; tensor leaves travel as they are, every other leaf is pickled into a
``uint8`` tensor ``[8-byte little-endian length | pickle | zero padding]`` whose capacity only grows, so
shapes stay constant between micro batches.  The first exchange is preceded by the pickled *meta
tree* (shape, dtype, requires_grad per leaf); afterwards the meta is assumed unchanged unless
``use_continuous_recommunication`` is set, in which case a one-element "meta changed" flag precedes
every exchange.  Gradients travel back for exactly the leaves that require grad, in leaf order.

All leaves of one exchange are posted as a single ``batch_isend_irecv`` group (one NCCL group launch
instead of one blocking send per leaf).  Transfers overlap compute in both directions:

* sends are not waited for where they are issued: the handles (and the tensors they read) are kept until
  the next send on the same link or ``drain()``, so the compute stream never stalls behind an outgoing copy;
* receives can be posted ahead of time (``post_recv`` for activations, ``post_recv_grad`` for gradients), which
  the schedule loop does as soon as the previous compute instruction has been enqueued; ``recv_data`` /
  ``recv_grad`` then only wait for them.

Activations and gradients of one link travel over different process groups (``group`` / ``grad_group``): each has
its own communicator and stream, so a receive that was posted early and is still waiting for its sender cannot
hold up a send in the other direction between the same two ranks.
"""

from __future__ import annotations

import pickle
from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.distributed as dist
from torch.utils import _pytree as pytree

from ....parallel.topology import Topology

_LEN_BYTES = 8


@dataclass
class LeafMeta:
    is_tensor: bool
    shape: tuple[int, ...]
    dtype: torch.dtype
    requires_grad: bool


def _encode_object(obj: Any, capacity: int, device: torch.device) -> torch.Tensor:
    raw = pickle.dumps(obj)
    need = _LEN_BYTES + len(raw)
    capacity = max(capacity, need)
    buf = bytearray(capacity)
    buf[:_LEN_BYTES] = len(raw).to_bytes(_LEN_BYTES, "little")
    buf[_LEN_BYTES:need] = raw
    return torch.frombuffer(buf, dtype=torch.uint8).clone().to(device)


def _decode_object(t: torch.Tensor) -> Any:
    raw = t.cpu().numpy().tobytes()
    n = int.from_bytes(raw[:_LEN_BYTES], "little")
    return pickle.loads(raw[_LEN_BYTES:_LEN_BYTES + n])


def _run(ops: list) -> None:
    if not ops:
        return
    for work in dist.batch_isend_irecv(ops):
        work.wait()


def _start(ops: list) -> list:
    return dist.batch_isend_irecv(ops) if ops else []


class PipeCommunicator:
    def __init__(self, local_device: torch.device, recv_grads: bool, recv_data: bool,
                 use_continuous_recommunication: bool, group: Any = None, peer_send: Optional[int] = None,
                 peer_recv: Optional[int] = None, grad_group: Any = None):
        """
        ``peer_send``: global rank data is sent to (and gradients are received from);
        ``peer_recv``: global rank data is received from (and gradients are sent to);
        ``group`` / ``grad_group``: process groups that carry the data and the gradients (default: the world group).
        """
        self.local_device = local_device
        self.can_recv_grads = recv_grads
        self.can_recv_data = recv_data
        self.use_continuous_recommunication = use_continuous_recommunication
        self.group = group
        self.grad_group = grad_group if grad_group is not None else group
        self.peer_send = peer_send
        self.peer_recv = peer_recv
        # Negotiated structure per channel: a training step and an evaluation step send differently flagged trees
        # (gradients wanted or not) over the same link; both sides switch channel together, so nothing extra is sent.
        self.channel = "train"
        self._state: dict[str, dict[str, Any]] = {}
        self._posted: Optional[tuple[list[torch.Tensor], list]] = None
        self._posted_grad: Optional[tuple[list[torch.Tensor], list[torch.Tensor], list]] = None
        self._sends_in_flight: list[tuple[list, list[torch.Tensor]]] = []

    def reset_communication_meta(self) -> None:
        self.drain()
        self._state = {}
        self._posted = None
        self._posted_grad = None

    # ------------------------------------------------------------------ sends in flight
    def _send_async(self, tensors: list[torch.Tensor], peer: int, group: Any) -> None:
        """Issue the sends and return at once.  The previous batch on this link is retired first (it has long
        finished; on a GPU this only orders the stream after it), so at most one batch of handles is kept."""
        self.drain()
        works = _start([dist.P2POp(dist.isend, t, peer, group=group) for t in tensors])
        if works:
            self._sends_in_flight.append((works, tensors))

    def drain(self) -> None:
        """Wait for outgoing transfers that were issued without waiting (end of a step, before shapes change)."""
        for works, _tensors in self._sends_in_flight:
            for w in works:
                w.wait()
        self._sends_in_flight = []

    def _channel_state(self) -> dict[str, Any]:
        st = self._state.get(self.channel)
        if st is None:
            st = self._state[self.channel] = dict(sent_meta=None, sent_spec=None, recv_meta=None, recv_spec=None,
                                                  obj_capacity={})
        return st

    _sent_meta = property(lambda self: self._channel_state()["sent_meta"],
                          lambda self, v: self._channel_state().__setitem__("sent_meta", v))
    _sent_spec = property(lambda self: self._channel_state()["sent_spec"],
                          lambda self, v: self._channel_state().__setitem__("sent_spec", v))
    _recv_meta = property(lambda self: self._channel_state()["recv_meta"],
                          lambda self, v: self._channel_state().__setitem__("recv_meta", v))
    _recv_spec = property(lambda self: self._channel_state()["recv_spec"],
                          lambda self, v: self._channel_state().__setitem__("recv_spec", v))
    _obj_capacity = property(lambda self: self._channel_state()["obj_capacity"])

    # ------------------------------------------------------------------ data: sender side
    def _to_wire(self, data: Any) -> tuple[list[torch.Tensor], list[LeafMeta], Any]:
        leaves, spec = pytree.tree_flatten(data)
        tensors: list[torch.Tensor] = []
        meta: list[LeafMeta] = []
        for i, leaf in enumerate(leaves):
            if isinstance(leaf, torch.Tensor):
                t = leaf.detach().contiguous()
                meta.append(LeafMeta(True, tuple(t.shape), t.dtype, bool(leaf.requires_grad)))
            else:
                t = _encode_object(leaf, self._obj_capacity.get(i, 0), self.local_device)
                self._obj_capacity[i] = t.numel()
                meta.append(LeafMeta(False, tuple(t.shape), t.dtype, False))
            tensors.append(t)
        return tensors, meta, spec

    def _send_meta(self, meta: list[LeafMeta], spec: Any) -> None:
        blob = _encode_object((meta, pytree.treespec_dumps(spec)), 0, self.local_device)
        n = torch.tensor([blob.numel()], dtype=torch.int64, device=self.local_device)
        dist.send(n, self.peer_send, group=self.group)
        dist.send(blob, self.peer_send, group=self.group)

    def send_data(self, data: Any) -> None:
        assert self.peer_send is not None
        tensors, meta, spec = self._to_wire(data)
        changed = self._sent_meta is None or meta != self._sent_meta or spec != self._sent_spec
        if self._sent_meta is None:
            self._send_meta(meta, spec)
        elif self.use_continuous_recommunication:
            flag = torch.tensor([1 if changed else 0], dtype=torch.int64, device=self.local_device)
            dist.send(flag, self.peer_send, group=self.group)
            if changed:
                self._send_meta(meta, spec)
        else:
            assert not changed, (
                "the structure of the data sent between pipeline stages changed; enable "
                "use_continuous_recommunication to renegotiate shapes on every exchange"
            )
        self._sent_meta, self._sent_spec = meta, spec
        self._send_async(tensors, self.peer_send, self.group)

    # ------------------------------------------------------------------ data: receiver side
    def _recv_meta_blob(self) -> None:
        n = torch.zeros(1, dtype=torch.int64, device=self.local_device)
        dist.recv(n, self.peer_recv, group=self.group)
        blob = torch.zeros(int(n.item()), dtype=torch.uint8, device=self.local_device)
        dist.recv(blob, self.peer_recv, group=self.group)
        self._recv_meta, spec = _decode_object(blob)
        self._recv_spec = pytree.treespec_loads(spec)

    def _negotiate_recv(self) -> None:
        if self._recv_meta is None:
            self._recv_meta_blob()
        elif self.use_continuous_recommunication:
            flag = torch.zeros(1, dtype=torch.int64, device=self.local_device)
            dist.recv(flag, self.peer_recv, group=self.group)
            if int(flag.item()) == 1:
                self._recv_meta_blob()

    def post_recv(self) -> bool:
        """Post the receives of the next exchange now; ``recv_data`` later only waits for them.  Possible once the
        structure of the data is known (after the first exchange) and fixed (no per-exchange renegotiation)."""
        assert self.peer_recv is not None
        if self._posted is not None or self._recv_meta is None or self.use_continuous_recommunication:
            return False
        bufs = [torch.empty(m.shape, dtype=m.dtype, device=self.local_device) for m in self._recv_meta]
        works = _start([dist.P2POp(dist.irecv, b, self.peer_recv, group=self.group) for b in bufs])
        self._posted = (bufs, works)
        return True

    def recv_data(self) -> Any:
        assert self.can_recv_data and self.peer_recv is not None
        if self._posted is not None:
            bufs, works = self._posted
            self._posted = None
            for w in works:
                w.wait()
        else:
            self._negotiate_recv()
            assert self._recv_meta is not None
            bufs = [torch.empty(m.shape, dtype=m.dtype, device=self.local_device) for m in self._recv_meta]
            _run([dist.P2POp(dist.irecv, b, self.peer_recv, group=self.group) for b in bufs])
        leaves: list[Any] = []
        for m, b in zip(self._recv_meta, bufs):  # type: ignore[arg-type]
            if m.is_tensor:
                if m.requires_grad:
                    b.requires_grad_(True)
                leaves.append(b)
            else:
                leaves.append(_decode_object(b))
        return pytree.tree_unflatten(leaves, self._recv_spec)

    # ------------------------------------------------------------------ gradients
    def send_grad(self, data: Any) -> None:
        """Send ``.grad`` of every leaf of the received input tree that requires grad."""
        assert self.peer_recv is not None
        leaves, _ = pytree.tree_flatten(data)
        ops = []
        for leaf in leaves:
            if isinstance(leaf, torch.Tensor) and leaf.requires_grad:
                g = leaf.grad if leaf.grad is not None else torch.zeros_like(leaf)
                ops.append(g.contiguous())
        self._send_async(ops, self.peer_recv, self.grad_group)

    def recv_grad(self, data: Any) -> tuple[list[torch.Tensor], list[torch.Tensor]]:
        """For the output tree that was sent, receive gradients; returns (tensors, grads) for autograd."""
        assert self.can_recv_grads and self.peer_send is not None
        tensors = self._grad_leaves(data)
        if self._posted_grad is not None:
            posted_for, grads, works = self._posted_grad
            self._posted_grad = None
            assert len(posted_for) == len(tensors) and all(a is b for a, b in zip(posted_for, tensors)), (
                "gradient receives were posted for another micro batch than the one now asked for"
            )
            for w in works:
                w.wait()
            return tensors, grads
        grads = [torch.empty_like(t, memory_format=torch.contiguous_format) for t in tensors]
        _run([dist.P2POp(dist.irecv, g, self.peer_send, group=self.grad_group) for g in grads])
        return tensors, grads

    @staticmethod
    def _grad_leaves(data: Any) -> list[torch.Tensor]:
        leaves, _ = pytree.tree_flatten(data)
        return [leaf for leaf in leaves if isinstance(leaf, torch.Tensor) and leaf.requires_grad]

    def post_recv_grad(self, data: Any) -> bool:
        """Post the receives for the gradients of the output tree ``data`` now; the matching ``recv_grad(data)`` only
        waits.  Returns False (nothing posted) while an earlier posting is still outstanding."""
        assert self.can_recv_grads and self.peer_send is not None
        if self._posted_grad is not None:
            return False
        tensors = self._grad_leaves(data)
        grads = [torch.empty_like(t, memory_format=torch.contiguous_format) for t in tensors]
        works = _start([dist.P2POp(dist.irecv, g, self.peer_send, group=self.grad_group) for g in grads])
        self._posted_grad = (tensors, grads, works)
        return True


class ModelParallelCommunicator:
    """Synchronises a pytree from one rank of a tensor-parallel group to the others by broadcast
    (utility with the role of src/scaling/core/nn/parallel_module/communicator.py:495-737)."""

    def __init__(self, topology: Topology, src_model_parallel_rank: int = 0):
        self.topology = topology
        self.src = topology.get_global_rank(model_parallel_rank=src_model_parallel_rank)
        self.is_src = topology.model_parallel_rank == src_model_parallel_rank

    def sync_data(self, data: Any = None) -> Any:
        group = self.topology.model_parallel_group
        dev = self.topology.device
        if self.topology.model_parallel_size == 1:
            return data
        if self.is_src:
            leaves, spec = pytree.tree_flatten(data)
            meta = [
                LeafMeta(True, tuple(x.shape), x.dtype, bool(x.requires_grad)) if isinstance(x, torch.Tensor) else x
                for x in leaves
            ]
            box = [(meta, spec)]
        else:
            box = [None]
        dist.broadcast_object_list(box, src=self.src, group=group, device=dev)
        meta, spec = box[0]
        out = []
        idx = 0
        for m in meta:
            if isinstance(m, LeafMeta):
                if self.is_src:
                    t = leaves[idx].detach().to(dev).contiguous()
                else:
                    t = torch.empty(m.shape, dtype=m.dtype, device=dev)
                dist.broadcast(t, src=self.src, group=group)
                out.append(t)
            else:
                out.append(m)
            idx += 1
        return pytree.tree_unflatten(out, spec)
