"""Helpers for multi-process tests: N local ranks with the gloo backend on CPU (or nccl on GPUs)."""

from __future__ import annotations

import os
import socket
import traceback
from contextlib import closing
from typing import Any, Callable

import torch
import torch.multiprocessing as mp

# generous: a loaded test machine must not look like a hung rank (SB200_TEST_TIMEOUT_S overrides)
PROCESS_TIMEOUT = int(os.environ.get("SB200_TEST_TIMEOUT_S", "300"))


def find_free_port() -> int:
    with closing(socket.socket(socket.AF_INET, socket.SOCK_STREAM)) as s:
        s.bind(("127.0.0.1", 0))
        return int(s.getsockname()[1])


def _worker(rank: int, world_size: int, port: int, fn: Callable, kwargs: dict, results: Any, device: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world_size), RANK=str(rank),
                      LOCAL_SLOT=str(rank))
    torch.set_num_threads(1)
    try:
        results[rank] = ("ok", fn(rank=rank, world_size=world_size, port=port, device=device, **kwargs))
    except BaseException:  # noqa: BLE001 - report everything to the parent
        results[rank] = ("error", traceback.format_exc())
    finally:
        import gc

        import torch.distributed as dist

        # captured CUDA graphs pin communicators: collect the finished run's objects before the teardown
        gc.collect()
        if torch.cuda.is_available() and device == "cuda":
            torch.cuda.synchronize()
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def dist_launcher(fn: Callable, world_size: int, device: str = "cpu", **kwargs: Any) -> list[Any]:
    """Run ``fn(rank, world_size, port, device, **kwargs)`` on ``world_size`` spawned ranks; return their results."""
    port = find_free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        results = manager.dict()
        procs = [ctx.Process(target=_worker, args=(r, world_size, port, fn, kwargs, results, device)) for r in range(world_size)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(PROCESS_TIMEOUT)
        hung = [i for i, p in enumerate(procs) if p.is_alive()]
        for p in procs:
            if p.is_alive():
                p.kill()
        out = dict(results)
    assert not hung, f"ranks {hung} did not finish within {PROCESS_TIMEOUT}s"
    errors = {r: v[1] for r, v in out.items() if v[0] == "error"}
    assert not errors, "rank failures:\n" + "\n".join(f"[rank {r}]\n{tb}" for r, tb in errors.items())
    missing = [r for r in range(world_size) if r not in out]
    assert not missing, f"ranks {missing} exited without a result"
    return [out[r][1] for r in range(world_size)]
