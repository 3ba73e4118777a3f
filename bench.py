"""Headline benchmark: training tokens/s of the 125M decoder (12 layers, hidden 768, 12 heads, vocab 32768,
pre-LayerNorm, GELU MLP 3072, RoPE, causal attention), seq 2048, micro batch 8 per GPU, bf16 with fp32 master
weights, data parallel over N GPUs with ZeRO-1, AdamW - seeded synthetic token ids, random-init weights.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference installed under baseline/_ref

Prints ONE json line on rank 0.  ``value`` is the whole-job tokens/s with inputs already on the device;
``e2e.value`` is measured through the public training API (``ParallelModule.train_step`` fed by the
``DataLoader``) and includes, per step, the host-to-device copy of the batch from pinned memory and the
device-to-host read of the loss.  Times are CUDA-event times, max over ranks; SM clocks and throttle reasons are
sampled with nvidia-smi during the timed region.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
MODEL = dict(vocab_size=32768, hidden_size=768, num_layers=12, num_attention_heads=12, sequence_length=2048,
             mlp_factor=4.0)
MICRO_BATCH = 8


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    return p.parse_args()


# ---------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return

        def pump() -> None:
            assert self.proc is not None and self.proc.stdout is not None
            for line in self.proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "", 1).isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "", 1).isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def dist_env(args: argparse.Namespace) -> tuple[int, int, int]:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    local = int(os.environ.get("LOCAL_RANK", os.environ.get("LOCAL_SLOT", str(rank))))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs a torchrun launch with {args.gpus} ranks (WORLD_SIZE is {world})")
    return rank, world, local


def result_line(args, world, tokens_per_step, dev_ms, e2e_ms, clocks, launches, h2d, d2h, impl) -> dict:
    value = tokens_per_step / (dev_ms / 1000.0)
    e2e = tokens_per_step / (e2e_ms / 1000.0)
    return {
        "metric": "train tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": impl,
        "config": {"model": "decoder-125M (12L, h768, 12 heads, vocab 32768, LayerNorm, GELU, RoPE)",
                   "global_batch": MICRO_BATCH * world, "seq_len": MODEL["sequence_length"],
                   "parallelism": f"dp{world}" + ("+zero1" if True else ""), "micro_batch": MICRO_BATCH,
                   "l2": "inputs and activations per step exceed L2 (>1 GB touched per step)"},
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
    }


# ---------------------------------------------------------------------------------------------- our arm
def run_ours(args: argparse.Namespace) -> None:
    import torch
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT))
    from scaling_b200.ops import _lib
    from scaling_b200.ops import functional as K
    from scaling_b200.parallel import Topology
    from scaling_b200.transformer import SyntheticTextDataset, TransformerConfig, TransformerContext, init_model, init_optimizer
    from scaling_b200.transformer.data import TextDatasetBatchBeforeSync
    from scaling_b200.transformer.model import metrics_aggregation_fn
    from scaling_b200.transformer.model.losses import create_loss_function
    from scaling_b200.core.data import DataLoader

    rank, world, local = dist_env(args)
    cfg = TransformerConfig.from_dict({
        "topology": {"world_size": world, "global_rank": rank, "local_slot": local, "model_parallel_size": 1,
                     "pipe_parallel_size": 1, "data_parallel_size": world, "micro_batch_size": MICRO_BATCH,
                     "gradient_accumulation_steps": 1},
        "optimizer": {"zero": True, "gradient_clipping": 1.0, "beta1": 0.9, "beta2": 0.95},
        "training_groups": [{"group_name": "all", "weight_decay": 0.1,
                             "learning_rate_scheduler": {"learning_rate": 3e-4, "learning_rate_decay_style": "constant"}}],
        "transformer_architecture": dict(MODEL, precision="bfloat16", norm_type="layernorm", mlp_type="default",
                                         relative_position_embedding_type="rotary", weight_tying=False,
                                         masked_softmax={"kernel": "flash_attention"}, causal=True),
        "trainer": {"seed": 42},
    })
    topology = Topology(cfg.topology)
    context = TransformerContext(config=cfg, topology=topology)
    context.initialize(master_addr=os.environ["MASTER_ADDR"], master_port=os.environ["MASTER_PORT"], seed=42)
    model = init_model(context)
    optimizer = init_optimizer(context, model)
    loss_fn = create_loss_function(context, cfg.training.loss_function_config)
    seq = MODEL["sequence_length"]
    total_steps = 2 * (args.steps + args.warmup) + 2
    dataset = SyntheticTextDataset(n_samples=MICRO_BATCH * world * total_steps, sequence_length=seq,
                                   vocab_size=MODEL["vocab_size"], seed=42, low=1)
    loader = DataLoader(seed=42, consumed_samples=0, dataset=dataset, topology=topology, pin_memory=True)
    sync = SyntheticTextDataset.sync_batch_to_model_parallel
    dev = topology.device

    # device-resident batches for the kernel-only measurement
    staged = []
    for _ in range(args.steps + args.warmup):
        b = next(loader)
        staged.append(b.token_ids.to(dev))
    torch.cuda.synchronize()

    class Staged:
        def __init__(self):
            self.i = 0

        def __next__(self):
            ids = staged[self.i % len(staged)]
            self.i += 1
            return TextDatasetBatchBeforeSync(token_ids=ids)

    sync_staged = sync

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(n_warm, n_steps, dl, sync_fn) -> float:
        for _ in range(n_warm):
            model.train_step(dl, optimizer, sync_fn, loss_fn, metrics_aggregation_fn)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_steps):
            out = model.train_step(dl, optimizer, sync_fn, loss_fn, metrics_aggregation_fn)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / n_steps], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        assert out.loss is not None and out.loss == out.loss, "loss is NaN"
        return float(ms.item())

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    calls0 = None
    # kernel-only: inputs resident on the device
    for _ in range(args.warmup):
        model.train_step(Staged(), optimizer, sync_staged, loss_fn, metrics_aggregation_fn)
    st = Staged()
    barrier()
    calls0 = _lib.kernel_calls()
    dev_ms = timed(0, args.steps, st, sync_staged)
    launches = _lib.kernel_calls() - calls0
    # end to end: DataLoader -> pinned host memory -> H2D -> step -> loss D2H
    e2e_ms = timed(args.warmup, args.steps, loader, sync)
    clocks = sampler.stop() if rank == 0 else {}
    K.check_status()
    if rank == 0:
        tokens = MICRO_BATCH * seq * world
        h2d = MICRO_BATCH * (seq + 1) * 8
        line = result_line(args, world, tokens, dev_ms, e2e_ms, clocks, launches, h2d, 4, "ours")
        line["config"]["data_parallel_exchange"] = optimizer.data_parallel_exchange
        line["config"]["cuda_graph"] = bool(getattr(model, "_graph", None) is not None)
        print(json.dumps(line), flush=True)
    shutdown(model, world)


def shutdown(model, world: int) -> None:
    """Release captured graphs (they pin NCCL resources) and tear the process group down.  The result line is out
    already; should the teardown block on a communicator that a graph still references, leave after a grace period
    instead of holding the launcher until the process-group timeout."""
    import gc
    import threading

    import torch
    import torch.distributed as dist

    sys.stdout.flush()
    if world <= 1 or not dist.is_initialized():
        return
    dist.barrier()
    torch.cuda.synchronize()
    if model is not None and hasattr(model, "release_cuda_graph"):
        model.release_cuda_graph()
    gc.collect()
    torch.cuda.synchronize()
    timer = threading.Timer(20.0, lambda: os._exit(0))
    timer.daemon = True
    timer.start()
    dist.destroy_process_group()
    timer.cancel()


def main() -> None:
    args = parse_args()
    # a stuck collective would otherwise block until the process-group timeout: dump every thread's stack and exit
    watchdog = int(os.environ.get("SB200_BENCH_WATCHDOG_S", "900"))
    if watchdog > 0:
        import faulthandler

        faulthandler.dump_traceback_later(watchdog, exit=True)
    if args.impl == "reference":
        sys.path.insert(0, str(ROOT))
        from baseline.reference_arm import run_reference

        run_reference(args, MODEL, MICRO_BATCH, ClockSampler, dist_env, result_line)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
