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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
MODEL = dict(vocab_size=32768, hidden_size=768, num_layers=12, num_attention_heads=12, sequence_length=2048,
             mlp_factor=4.0)
MICRO_BATCH = 8

LLAMA = dict(norm_type="rms", mlp_type="swiglu", attention_bias=False, mlp_bias=False, attention_qkv_in_one=False,
             relative_position_embedding_type="rotary_complex")
LORA = {"name": "lora", "rank": 16, "alpha": 32, "parallel_modules": ["query", "key", "value", "dense"]}
# name -> (label, architecture, micro batch, global batch per step (None: micro x dp), tensor-parallel size,
#          pipeline stages, activation checkpointing, trains only the LoRA weights)
CONFIGS = {
    "125m": dict(label="decoder-125M (12L, h768, 12 heads, vocab 32768, LayerNorm, GELU, RoPE)",
                 arch=dict(MODEL, norm_type="layernorm", mlp_type="default", relative_position_embedding_type="rotary"),
                 micro=MICRO_BATCH, global_batch=None, mp=1, pp=1, ckpt="disabled", lora=False),
    "7b": dict(label="llama-7B (32L, h4096, 32q/8kv heads of 128, vocab 65536, RMSNorm, SwiGLU 11008, RoPE)",
               arch=dict(LLAMA, vocab_size=65536, hidden_size=4096, num_layers=32, num_attention_heads=32,
                         attention_num_kv_heads=8, sequence_length=4096, mlp_factor=11008 / 4096),
               micro=1, global_batch=64, mp=4, pp=1, ckpt="every_layer", lora=False),
    "7b_lora": dict(label="llama-7B frozen + LoRA r16 on q/k/v/o, seq 8192",
                    arch=dict(LLAMA, vocab_size=65536, hidden_size=4096, num_layers=32, num_attention_heads=32,
                              attention_num_kv_heads=8, sequence_length=8192, mlp_factor=11008 / 4096,
                              lora_config=LORA),
                    micro=1, global_batch=32, mp=8, pp=1, ckpt="every_layer", lora=True),
    "13b": dict(label="13B MQA (40L, h5120, 40q/1kv heads of 128, vocab 65536, RMSNorm, SwiGLU 13824, RoPE)",
                arch=dict(LLAMA, vocab_size=65536, hidden_size=5120, num_layers=40, num_attention_heads=40,
                          attention_num_kv_heads=1, sequence_length=4096, mlp_factor=13824 / 5120),
                micro=1, global_batch=32, mp=2, pp=2, ckpt="every_layer", lora=False),
}


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    p.add_argument("--config", type=str, default="125m", choices=sorted(CONFIGS),
                   help="model and layout; the tensor/pipeline sizes shrink to what --gpus allows")
    p.add_argument("--grad-accum", type=int, default=None,
                   help="micro batches per step and data-parallel rank (default: from the config's global batch)")
    p.add_argument("--layers", type=int, default=None, help="override the layer count (exploration only)")
    p.add_argument("--mp", type=int, default=None, help="override the config's tensor-parallel size")
    p.add_argument("--pp", type=int, default=None, help="override the config's number of pipeline stages")
    p.add_argument("--sequence-parallel", action="store_true",
                   help="shard the activations between the tensor-parallel linears over the tokens")
    return p.parse_args()


def layout(args: argparse.Namespace, world: int) -> dict:
    """Resolve the named config against the number of ranks: parallel sizes, accumulation steps, labels."""
    c = CONFIGS[args.config]
    if getattr(args, "mp", None) or getattr(args, "pp", None):
        c = dict(c, mp=args.mp or c["mp"], pp=args.pp or c["pp"])
    pp = c["pp"] if world % c["pp"] == 0 and world >= c["pp"] * min(c["mp"], 2) else 1
    mp = c["mp"]
    while mp > 1 and (world // pp) % mp:
        mp //= 2
    dp = world // (mp * pp)
    ga = args.grad_accum or (max(1, c["global_batch"] // (c["micro"] * dp)) if c["global_batch"] else 1)
    arch = dict(c["arch"])
    if args.layers:
        arch["num_layers"] = args.layers
    par = "+".join(f"{k}{v}" for k, v in (("tp", mp), ("pp", pp), ("dp", dp)) if v > 1 or k == "dp") + "+zero1"
    if getattr(args, "sequence_parallel", False) and mp > 1:
        par += "+sp"
    return dict(c, arch=arch, mp=mp, pp=pp, dp=dp, ga=ga, parallelism=par)


def model_flops_per_token(arch: dict, trains_base: bool) -> float:
    """Forward+backward model FLOPs per token (no recomputation counted): 6 per weight of the blocks and the head
    (4 when the base is frozen: no weight gradients), plus causal attention 6 * layers * seq * hidden."""
    h, L, s, V = arch["hidden_size"], arch["num_layers"], arch["sequence_length"], arch["vocab_size"]
    heads = arch["num_attention_heads"]
    kv = arch.get("attention_num_kv_heads") or heads
    d = h // heads
    attn = h * heads * d + 2 * h * kv * d + heads * d * h
    inner = int(round(arch.get("mlp_factor", 4.0) * h))
    mlp = (3 if arch.get("mlp_type") == "swiglu" else 2) * h * inner
    weights = L * (attn + mlp) + V * h
    return (6.0 if trains_base else 4.0) * weights + 6.0 * L * s * h


def measured_peak_tflops() -> tuple[float, str]:
    """Denominator of the reported MFU: the sustained bf16 matmul throughput measured on this pool's GPUs (the
    file the benchmark driver writes next to this script), else the sustained figure of an earlier measurement."""
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        return float(peaks["bf16_tflops_sustained"]), "bf16_tflops_sustained of measured"
    except Exception:
        return 1400.0, "1400 TFLOP/s sustained of fallback"


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


def result_line(args, world, tokens_per_step, dev_ms, e2e_ms, clocks, launches, h2d, d2h, impl, lay=None) -> dict:
    lay = lay or layout(args, world)
    value = tokens_per_step / (dev_ms / 1000.0)
    e2e = tokens_per_step / (e2e_ms / 1000.0)
    return {
        "metric": "train tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": impl,
        "config": {"model": lay["label"], "global_batch": lay["micro"] * lay["dp"] * lay["ga"],
                   "seq_len": lay["arch"]["sequence_length"], "parallelism": lay["parallelism"],
                   "micro_batch": lay["micro"], "gradient_accumulation_steps": lay["ga"],
                   "activation_checkpointing": lay["ckpt"],
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
    lay = layout(args, world)
    arch, micro, ga, dp = lay["arch"], lay["micro"], lay["ga"], lay["dp"]
    group = {"group_name": "all", "weight_decay": 0.1,
             "learning_rate_scheduler": {"learning_rate": 3e-4, "learning_rate_decay_style": "constant"}}
    if lay["lora"]:
        group = dict(group, group_name="lora", parameters_include=["lora"], weight_decay=0.0)
    cfg = TransformerConfig.from_dict({
        "topology": {"world_size": world, "global_rank": rank, "local_slot": local, "model_parallel_size": lay["mp"],
                     "pipe_parallel_size": lay["pp"], "data_parallel_size": dp, "micro_batch_size": micro,
                     "gradient_accumulation_steps": ga, "activation_checkpointing_type": lay["ckpt"],
                     "sequence_parallel": bool(args.sequence_parallel and lay["mp"] > 1)},
        "optimizer": {"zero": True, "gradient_clipping": 1.0, "beta1": 0.9, "beta2": 0.95},
        "training_groups": [group],
        "training": {"allow_missing_params_in_optimizer": True} if lay["lora"] else {},
        "transformer_architecture": dict(arch, precision="bfloat16", weight_tying=False,
                                         masked_softmax={"kernel": "flash_attention"}, causal=True),
        "trainer": {"seed": 42},
    })
    topology = Topology(cfg.topology)
    context = TransformerContext(config=cfg, topology=topology)
    context.initialize(master_addr=os.environ["MASTER_ADDR"], master_port=os.environ["MASTER_PORT"], seed=42)
    model = init_model(context)
    optimizer = init_optimizer(context, model)
    loss_fn = create_loss_function(context, cfg.training.loss_function_config)
    seq = arch["sequence_length"]
    total_steps = 2 * (args.steps + args.warmup) + 2
    dataset = SyntheticTextDataset(n_samples=micro * dp * ga * total_steps, sequence_length=seq,
                                   vocab_size=arch["vocab_size"], seed=42, low=1)
    loader = DataLoader(seed=42, consumed_samples=0, dataset=dataset, topology=topology, pin_memory=True) \
        if topology.is_io_rank else None
    sync = SyntheticTextDataset.sync_batch_to_model_parallel
    dev = topology.device

    # device-resident batches for the kernel-only measurement
    staged = []
    if loader is not None:
        for _ in range(min(args.steps + args.warmup, 8) * ga):
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
        assert out.loss is None or out.loss == out.loss, "loss is NaN"
        return float(ms.item())

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    calls0 = None
    # kernel-only: inputs resident on the device
    for _ in range(args.warmup):
        model.train_step(Staged() if staged else None, optimizer, sync_staged, loss_fn, metrics_aggregation_fn)
    st = Staged() if staged else None
    barrier()
    calls0 = _lib.kernel_calls()
    dev_ms = timed(0, args.steps, st, sync_staged)
    launches = _lib.kernel_calls() - calls0
    # end to end: DataLoader -> pinned host memory -> H2D -> step -> loss D2H
    e2e_ms = timed(args.warmup, args.steps, loader, sync)
    clocks = sampler.stop() if rank == 0 else {}
    K.check_status()
    if rank == 0:
        tokens = micro * seq * dp * ga
        h2d = micro * ga * (seq + 1) * 8
        line = result_line(args, world, tokens, dev_ms, e2e_ms, clocks, launches, h2d, 4 * ga, "ours", lay)
        tflops = model_flops_per_token(arch, not lay["lora"]) * line["value"] / world / 1e12
        peak, peak_name = measured_peak_tflops()
        line["details"] = {"data_parallel_exchange": optimizer.data_parallel_exchange,
                           "cuda_graph": model.cuda_graph_state(),
                           "model_tflops_per_gpu": round(tflops, 1),
                           "mfu": round(tflops / peak, 4), "mfu_denominator": peak_name}
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

        world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
        run_reference(args, layout(args, world), ClockSampler, dist_env, result_line)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
