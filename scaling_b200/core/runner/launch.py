"""Node launcher: starts one process per local slot and supervises them.

``python -m scaling_b200.core.runner.launch --resource_pool=<b64> --node_rank=N --master_addr=A
--master_port=P script --payload <b64>``.  Global ranks are assigned in pool order.  The first child
that exits non-zero takes the whole node down (every child is terminated, then killed), and
SIGINT/SIGTERM are fanned out, as in the reference (src/scaling/core/runner/launch.py:73-161).
"""

from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import time
from pathlib import Path
from typing import Any, Optional

from .launch_config import decode_base64

POLL_SECONDS = 0.2
GRACE_SECONDS = 5.0


def parse_args(argv: Optional[list[str]] = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="scaling_b200 node launcher")
    p.add_argument("--resource_pool", type=str, required=True, help="base64 json {'nodes': [...], 'world_size': n}")
    p.add_argument("--node_rank", type=int, default=0)
    p.add_argument("--master_addr", type=str, default="127.0.0.1")
    p.add_argument("--master_port", type=int, default=29500)
    p.add_argument("script", type=str)
    p.add_argument("--payload", type=str, default=None)
    return p.parse_args(argv)


def local_assignment(pool: dict[str, Any], node_rank: int) -> tuple[list[int], list[int], int]:
    """(slots, global ranks) of node ``node_rank`` and the world size implied by the pool."""
    next_rank = 0
    slots: list[int] = []
    ranks: list[int] = []
    for i, node in enumerate(pool["nodes"]):
        n = len(node["slots"])
        if i == node_rank:
            slots = list(node["slots"])
            ranks = list(range(next_rank, next_rank + n))
        next_rank += n
    assert next_rank == pool["world_size"], "derived world size differs from communicated world size"
    return slots, ranks, next_rank


def _terminate(children: list[subprocess.Popen]) -> None:
    for c in children:
        if c.poll() is None:
            try:
                c.terminate()
            except Exception:
                pass
    deadline = time.time() + GRACE_SECONDS
    for c in children:
        remaining = max(0.0, deadline - time.time())
        try:
            c.wait(timeout=remaining)
        except Exception:
            try:
                c.kill()
            except Exception:
                pass


def script_command(script: str) -> tuple[list[str], Optional[str]]:
    """How to start ``script``: a file that belongs to a package (``__init__.py`` in its folder and above) runs as
    ``python -m package.module`` with the package's parent folder on the import path, so that its relative imports
    work; any other file runs as a plain script."""
    path = Path(script).resolve()
    if path.suffix != ".py" or not (path.parent / "__init__.py").is_file():
        return [sys.executable, "-u", script], None
    parts = [path.stem]
    folder = path.parent
    while (folder / "__init__.py").is_file():
        parts.append(folder.name)
        folder = folder.parent
    return [sys.executable, "-u", "-m", ".".join(reversed(parts))], str(folder)


def main(argv: Optional[list[str]] = None) -> int:
    args = parse_args(argv)
    pool = decode_base64(args.resource_pool)
    slots, ranks, world_size = local_assignment(pool, args.node_rank)
    env = os.environ.copy()
    env.update(MASTER_ADDR=args.master_addr, MASTER_PORT=str(args.master_port), WORLD_SIZE=str(world_size))
    children: list[subprocess.Popen] = []
    base_cmd, import_root = script_command(args.script)
    if import_root is not None:
        env["PYTHONPATH"] = import_root + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
    for slot, rank in zip(slots, ranks):
        child_env = dict(env, RANK=str(rank), LOCAL_SLOT=str(slot))
        cmd = list(base_cmd)
        if args.payload is not None:
            cmd += ["--payload", args.payload]
        children.append(subprocess.Popen(cmd, env=child_env))

    def on_signal(signum: int, frame: Any) -> None:
        _terminate(children)
        sys.exit(128 + signum)

    signal.signal(signal.SIGINT, on_signal)
    signal.signal(signal.SIGTERM, on_signal)

    alive = list(children)
    while alive:
        still = []
        for c in alive:
            rc = c.poll()
            if rc is None:
                still.append(c)
            elif rc != 0:
                _terminate(children)
                return rc if rc > 0 else 1
        alive = still
        if alive:
            time.sleep(POLL_SECONDS)
    return 0


if __name__ == "__main__":
    sys.exit(main())
