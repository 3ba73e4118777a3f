"""Host-side model of the flag protocol of the fused tensor-parallel GEMM kernel (``sb200_gemm_tp``).

Every rank is a group of Python threads over shared numpy arrays that stand for the symmetric buffers: per CTA one
"compute" thread (producer + MMA + epilogue of the kernel) and one "helper" thread (the reducer / gather warps).  The
model keeps exactly the kernel's ordering rules and nothing of its arithmetic detail:

* flags only grow: a flag word holds the epoch (launch number) of the last launch that set it, a wait is ``>= epoch``;
* all-reduce / reduce-scatter: a tile's partial product is published to the tile's owner, the owner reduces once all
  ranks have published; an all-reduce launch (whose output is written by the peers) ends only after every rank has
  reported the end of its reductions;
* all-gather: a row block is pushed in column groups, each with its own flag; the tile loads of a block wait for all
  its groups;
* the partial products / the gathered operand live in two buffers that consecutive launches use in turn, so a
  buffer is rewritten two launches after it was filled; no rank can finish a launch before every peer has entered
  it, hence whoever read the buffer is done by then.  The first launch of a count (``sync_entry``) starts at buffer 0
  and first waits until every rank has entered it (a captured training step is replayed from its first launch
  whatever buffer its last launch used);
* between launches a rank may read its gathered operand (linears that share an input): nobody may write it then.

Random delays shuffle the interleavings.  The model checks the results against numpy, that no wait runs out, and that
a rank's gathered operand does not change between the end of a launch and the rank's entry into the next one.  It
checks the protocol logic only: memory-model fences are a matter of the kernel source.
"""

from __future__ import annotations

import random
import threading
import time
from typing import Optional

import numpy as np

ALLREDUCE, REDUCE_SCATTER, ALLGATHER = 0, 1, 2
BM = 4  # rows of a tile / row block in the model


class ProtocolError(AssertionError):
    pass


class Workspace:
    """Symmetric buffers of a group of ``W`` ranks (index = rank) plus each rank's local words."""

    def __init__(self, W: int, max_elements: int, flag_stride: int = 64):
        self.W = W
        self.stride = flag_stride
        self.half_elems = max_elements
        self.partial = [np.zeros(2 * max_elements, dtype=np.float64) for _ in range(W)]  # two buffers used in turn
        self.out = [np.zeros(max_elements, dtype=np.float64) for _ in range(W)]
        self.flags = [np.zeros((W + 2) * flag_stride, dtype=np.int64) for _ in range(W)]
        self.epoch = [0] * W
        self.done_ctas = [0] * W
        self.lock = [threading.Lock() for _ in range(W)]  # the atomicAdd on done_ctas
        self.failed = threading.Event()  # a rank of the model found a violation: the others stop waiting for it


def _wait(flags: np.ndarray, index: int, value: int, timeout: float, what: str,
          failed: Optional[threading.Event] = None) -> None:
    deadline = time.monotonic() + timeout
    while flags[index] < value:
        if time.monotonic() > deadline:
            raise ProtocolError(f"wait ran out: {what}")
        if failed is not None and failed.is_set():
            raise ProtocolError(f"stopped while waiting ({what}): another rank reported a violation")
        time.sleep(0)


def _jitter(rng: random.Random, scale: float) -> None:
    if scale > 0:
        time.sleep(rng.random() * scale)


def launch(ws: Workspace, rank: int, mode: int, a: np.ndarray, b: np.ndarray, ctas: int, seed: int,
           jitter: float = 2e-4, timeout: float = 20.0, groups: int = 2, half: int = 0,
           sync_entry: bool = False) -> Optional[np.ndarray]:
    """One rank's launch.  ``a``: ``[M, K]`` (modes 0, 1) or this rank's ``[M / W, K]`` shard (mode 2); ``b``: ``[K, N]``.
    Returns the reduced ``[M, N]`` (mode 0), this rank's rows of it (mode 1) or the local product (mode 2)."""
    W = ws.W
    epoch = ws.epoch[rank] + 1
    stride = ws.stride
    N = b.shape[1]
    K = b.shape[0]
    M = a.shape[0] * (W if mode == ALLGATHER else 1)
    assert M % (BM * W) == 0
    m_tiles = M // BM
    shard_rows = M // W
    shift = 0
    if mode == REDUCE_SCATTER:
        shift = ((rank + 1) % W) * (m_tiles // W)
    elif mode == ALLGATHER:
        shift = rank * (m_tiles // W)
    result = np.zeros((M, N)) if mode != REDUCE_SCATTER else np.zeros((shard_rows, N))
    hoff = half * ws.half_elems

    def buffer_of(q: int, cols: int) -> np.ndarray:
        return ws.partial[q][hoff:hoff + M * cols].reshape(M, cols)

    partial = buffer_of(rank, N)
    errors: list[BaseException] = []
    if sync_entry:  # every CTA waits (thread 0 of the kernel, before the roles start); CTA 0 signals
        for q in range(W):
            ws.flags[q][(W + 1) * stride + rank] = epoch
        for q in range(W):
            _wait(ws.flags[rank], (W + 1) * stride + q, epoch, timeout, f"rank {rank}: entry of rank {q}", ws.failed)

    def tile_of(cta: int, i: int) -> int:
        return (cta + i * ctas + shift) % m_tiles

    def owner_of(tile: int) -> int:
        return (tile * BM) // shard_rows if mode == REDUCE_SCATTER else tile % W

    def compute(cta: int) -> None:
        rng = random.Random(seed * 1000 + cta)
        try:
            for i in range((m_tiles - cta + ctas - 1) // ctas):
                tile = tile_of(cta, i)
                rows = slice(tile * BM, (tile + 1) * BM)
                if mode == ALLGATHER:
                    src = (tile * BM) // shard_rows
                    rb = (tile * BM - src * shard_rows) // BM
                    for g in range(groups):  # tile loads wait for every column group of the row block
                        _wait(ws.flags[rank], src * stride + rb * groups + g, epoch, timeout,
                              f"rank {rank} rows of rank {src} block {rb} group {g}", ws.failed)
                    result[rows] = buffer_of(rank, K)[rows] @ b
                else:
                    _jitter(rng, jitter)
                    partial[rows] = a[rows] @ b  # epilogue: the partial tile, then the flag at the owner
                    ws.flags[owner_of(tile)][rank * stride + tile] = epoch
        except BaseException as e:  # noqa: BLE001
            errors.append(e)

    def helper(cta: int) -> None:
        rng = random.Random(seed * 1000 + 500 + cta)
        try:
            if mode == ALLGATHER:
                blocks = shard_rows // BM
                cw = (K + groups - 1) // groups
                for item in range(cta, blocks * groups, ctas):
                    rb, g = divmod(item, groups)
                    _jitter(rng, jitter)
                    cols = slice(g * cw, min(K, (g + 1) * cw))
                    for q in range(W):
                        dst = buffer_of(q, K)
                        dst[rank * shard_rows + rb * BM: rank * shard_rows + (rb + 1) * BM, cols] = \
                            a[rb * BM:(rb + 1) * BM, cols]
                    for q in range(W):
                        ws.flags[q][rank * stride + item] = epoch
                return
            for i in range((m_tiles - cta + ctas - 1) // ctas):
                tile = tile_of(cta, i)
                if owner_of(tile) != rank:
                    continue
                for q in range(W):
                    _wait(ws.flags[rank], q * stride + tile, epoch, timeout, f"rank {rank}: tile {tile} of rank {q}",
                          ws.failed)
                _jitter(rng, jitter)
                rows = slice(tile * BM, (tile + 1) * BM)
                total = sum(buffer_of(q, N)[rows] for q in range(W))  # rank order
                if mode == REDUCE_SCATTER:
                    result[tile * BM - rank * shard_rows: (tile + 1) * BM - rank * shard_rows] = total
                else:
                    for q in range(W):
                        ws.out[q][:M * N].reshape(M, N)[rows] = total
        except BaseException as e:  # noqa: BLE001
            errors.append(e)

    def cta_main(cta: int) -> None:
        threads = [threading.Thread(target=compute, args=(cta,)), threading.Thread(target=helper, args=(cta,))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        with ws.lock[rank]:
            ws.done_ctas[rank] += 1
            last = ws.done_ctas[rank] == ctas
            if last:
                ws.done_ctas[rank] = 0
        if last:  # the last CTA advances the epoch; after an all-reduce it first tells and waits for every rank
            try:
                if mode == ALLREDUCE:
                    for q in range(W):
                        ws.flags[q][W * stride + rank] = epoch
                    for q in range(W):
                        _wait(ws.flags[rank], W * stride + q, epoch, timeout, f"rank {rank}: end of rank {q}",
                              ws.failed)
                ws.epoch[rank] = epoch
            except BaseException as e:  # noqa: BLE001
                errors.append(e)

    cta_threads = [threading.Thread(target=cta_main, args=(c,)) for c in range(ctas)]
    for t in cta_threads:
        t.start()
    for t in cta_threads:
        t.join()
    if errors:
        raise errors[0]
    if mode == ALLREDUCE:
        return ws.out[rank][:M * N].reshape(M, N).copy()
    return result


def run_sequence(W: int, modes: list[int], seed: int = 0, ctas: int = 3, M: int = 24, N: int = 5, K: int = 6,
                 jitter: float = 2e-4, alternate: bool = True, slow_reader: Optional[int] = None,
                 step_length: Optional[int] = None) -> None:
    """All ranks run the same sequence of launches (as a training step does) with their own operands and random
    delays between launches; after an all-gather launch a rank keeps reading its gathered operand until it enters
    its next launch and checks that it does not change.  Every ``step_length`` launches (default: never again after
    the first) the buffer alternation starts anew with a launch that synchronises on entry, as at the start of a
    training step.  ``alternate=False`` keeps every launch in buffer 0 (to show what the alternation prevents).
    Raises :class:`ProtocolError` on any violation."""
    M = (M + BM * W - 1) // (BM * W) * (BM * W)
    ws = Workspace(W, max(M * N, M * K))
    rng0 = np.random.default_rng(seed)
    operands = []
    for step, mode in enumerate(modes):
        if mode == ALLGATHER:
            shards = [rng0.standard_normal((M // W, K)) for _ in range(W)]
            b = [rng0.standard_normal((K, N))] * W
            full = np.concatenate(shards, axis=0)
            expect = [full @ b[0]] * W
            operands.append((shards, b, expect, full))
        else:
            a = [rng0.standard_normal((M, K)) for _ in range(W)]
            b = [rng0.standard_normal((K, N)) for _ in range(W)]
            total = sum(x @ y for x, y in zip(a, b))
            expect = [total if mode == ALLREDUCE else total[r * (M // W):(r + 1) * (M // W)] for r in range(W)]
            operands.append((a, b, expect, None))
    failures: list[BaseException] = []

    def rank_main(rank: int) -> None:
        rng = random.Random(seed * 77 + rank)
        try:
            for step, mode in enumerate(modes):
                a, b, expect, full = operands[step]
                count = step % step_length if step_length else step
                half = count & 1 if alternate else 0
                got = launch(ws, rank, mode, a[rank], b[rank], ctas, seed * 131 + step * 7 + rank, jitter,
                             half=half, sync_entry=count == 0)
                if not np.allclose(got, expect[rank]):
                    raise ProtocolError(f"rank {rank} launch {step} (mode {mode}): wrong result")
                if mode == ALLGATHER:
                    # linears that share the input read the gathered operand now, while peers may already be ahead
                    for _ in range(3):
                        _jitter(rng, 4 * jitter)
                        if rank == slow_reader:
                            time.sleep(0.05)
                        base = half * ws.half_elems
                        if not np.array_equal(ws.partial[rank][base:base + M * K].reshape(M, K), full):
                            raise ProtocolError(f"rank {rank}: gathered operand changed after launch {step}")
                else:
                    _jitter(rng, 4 * jitter)
        except BaseException as e:  # noqa: BLE001
            failures.append(e)
            ws.failed.set()

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(W)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if failures:
        first = [f for f in failures if "another rank reported" not in str(f)]
        raise (first or failures)[0]
