"""Sustained-loop timings of the tcgen05 GEMM on the linear-layer shapes of the 7B model (whole and on four
tensor-parallel ranks): forward (NT), input gradient (NN) and accumulating weight gradient (TN) for each tile shape
the kernel has, next to ``torch.matmul`` (cuBLAS) on the same operands.

    python -m benchmarks.gemm_shapes [--iters 60]

The GPU is first driven into its sustained state (power cap) with a few hundred large products; every figure is the
CUDA-event time of ``iters`` back-to-back launches divided by ``iters``.  Operands of one shape occupy 60 - 250 MB,
more than stays in L2 between launches.  One JSON line per shape: ``[microseconds, TFLOP/s]`` per variant.
"""

from __future__ import annotations

import argparse
import json
import sys

import torch

from scaling_b200.ops import functional as K

SHAPES = [  # name, tokens M, output features N, input features K
    ("dense 4096x4096x4096", 4096, 4096, 4096),
    ("qkv 4096x12288x4096", 4096, 12288, 4096),
    ("swiglu-in 4096x11008x4096", 4096, 11008, 4096),
    ("mlp-out 4096x4096x11008", 4096, 4096, 11008),
    ("tp4 mlp-in 4096x2752x4096", 4096, 2752, 4096),
    ("tp4 mlp-out 4096x4096x2752", 4096, 4096, 2752),
    ("tp4 qkv 4096x3072x4096", 4096, 3072, 4096),
    ("8k dense 8192x4096x4096", 8192, 4096, 4096),
]


def _time(fn, iters: int) -> float:
    for _ in range(10):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters * 1e3


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--iters", type=int, default=60)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        sys.exit("a CUDA device is required")
    dev, dt = "cuda", torch.bfloat16
    heat = torch.randn(8192, 8192, device=dev, dtype=dt)
    for _ in range(300):
        heat @ heat
    torch.cuda.synchronize()
    for name, M, N, Kd in SHAPES:
        x = torch.randn(M, Kd, device=dev, dtype=dt)
        w = torch.randn(N, Kd, device=dev, dtype=dt)
        dy = torch.randn(M, N, device=dev, dtype=dt)
        y = torch.empty(M, N, device=dev, dtype=dt)
        dx = torch.empty(M, Kd, device=dev, dtype=dt)
        dw = torch.zeros(N, Kd, device=dev, dtype=dt)
        flops = 2.0 * M * N * Kd
        row: dict = {"shape": name}

        def put(key: str, fn) -> None:
            t = _time(fn, args.iters)
            row[key] = [round(t, 1), round(flops / t / 1e6)]

        put("cublas_nt", lambda: torch.matmul(x, w.t(), out=y))
        for shape in (128, 256, 512):
            put(f"nt_{shape}", lambda: K.gemm(x, w, out=y, bn=shape, split=1))
        put("nt_auto", lambda: K.gemm(x, w, out=y))
        put("cublas_nn", lambda: torch.matmul(dy, w, out=dx))
        put("nn_auto", lambda: K.gemm(dy, w, b_mn=True, out=dx))
        put("cublas_tn", lambda: torch.matmul(dy.t(), x, out=dw))  # overwrites; ours accumulates (reads dw as well)
        for shape in (256, 512):
            put(f"tn_{shape}", lambda: K.gemm(dy, x, a_mn=True, b_mn=True, out=dw, accumulate=True, bn=shape, split=1))
        put("tn_auto", lambda: K.gemm(dy, x, a_mn=True, b_mn=True, out=dw, accumulate=True))
        K.check_status()
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
