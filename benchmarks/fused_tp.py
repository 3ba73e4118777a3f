"""Microbenchmark of the tensor-parallel GEMMs with in-kernel collectives against GEMM + NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m benchmarks.fused_tp [--multicast 0|1] [--iters 10]

For every shape, the row-parallel forms (``x [M, K / N_ranks] @ w^T`` followed by reduce-scatter or all-reduce) and the
column-parallel form (all-gather of ``[M / N_ranks, N]`` followed by a GEMM) are timed with CUDA events on the
launching stream, L2 flushed before every timed launch, median over ``--iters`` launches, maximum over ranks.  Rank 0
prints one JSON line per shape with the times in microseconds and the fused kernel's fraction of its roofline: the
slower of FLOPs / measured GEMM peak and bytes over NVLink / measured peer-copy bandwidth.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from scaling_b200.ops import functional as K
from scaling_b200.parallel.fused_tp import FusedTPWorkspace

GEMM_PEAK_FLOPS = 1.573e15  # measured cuBLAS bf16 burst on this part
LINK_BYTES_PER_S = 770e9    # measured peer copy, per direction

# (M tokens, N, K before the split): fc2 and attention output of the 125M decoder; MLP and attention output of the
# 7B model at 4096 and 8192 tokens, its output head (K = vocabulary)
SHAPES = [(16384, 768, 3072), (16384, 768, 768), (4096, 4096, 11008), (4096, 4096, 4096), (8192, 4096, 11008),
          (4096, 4096, 65536), (2048, 768, 768)]


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--multicast", type=int, default=1)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ws = FusedTPWorkspace(dist.group.WORLD, dev, 64 << 20, use_multicast=bool(args.multicast))

    def timeit(fn) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(args.iters):
            flush.zero_()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        t = torch.tensor(sorted(times)[len(times) // 2], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() * 1000.0

    for M, N, k_full in SHAPES:
        Kd = k_full // world // 8 * 8
        x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.02
        shard_out = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)

        def nccl_rs():
            dist.reduce_scatter_tensor(shard_out, K.gemm(x, w))

        def nccl_ar():
            dist.all_reduce(K.gemm(x, w))

        shard = torch.randn(M // world, N, device=dev, dtype=torch.bfloat16)
        w2 = torch.randn(Kd, N, device=dev, dtype=torch.bfloat16) * 0.02
        full = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

        def nccl_ag():
            dist.all_gather_into_tensor(full, shard)
            K.gemm(full, w2)

        flops = 2.0 * M * N * Kd
        frac = (world - 1) / world
        row = {
            "M": M, "N": N, "K_local": Kd, "ranks": world, "multicast": bool(args.multicast and ws.use_multicast),
            "gemm_us": timeit(lambda: K.gemm(x, w)),
            "rs_nccl_us": timeit(nccl_rs), "rs_fused_us": timeit(lambda: ws.gemm_reduce_scatter(x, w)),
            "ar_nccl_us": timeit(nccl_ar), "ar_fused_us": timeit(lambda: ws.gemm_allreduce(x, w)),
            "ag_nccl_us": timeit(nccl_ag), "ag_fused_us": timeit(lambda: ws.allgather_gemm(shard, w2)),
        }
        # bytes one GPU has to send: reduce-scatter (W-1)/W of the bf16 output, all-reduce twice that, all-gather
        # (W-1) copies of its shard (one with the switch's multicast)
        t_compute = flops / GEMM_PEAK_FLOPS * 1e6
        link = {"rs": frac * M * N * 2, "ar": 2 * frac * M * N * 2, "ag": (world - 1) * (M // world) * N * 2}
        for kind in ("rs", "ar", "ag"):
            roof = max(t_compute, link[kind] / LINK_BYTES_PER_S * 1e6)
            row[f"{kind}_roofline_fraction"] = round(roof / row[f"{kind}_fused_us"], 3)
        for key, val in row.items():
            if key.endswith("_us"):
                row[key] = round(val, 1)
        if rank == 0:
            print(json.dumps(row), flush=True)
    K.check_status()
    del ws
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
