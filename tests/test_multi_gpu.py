"""Multi-GPU paths on real devices (NCCL + the NVLink peer-memory kernels); skipped with fewer than two GPUs."""

import os
from pathlib import Path

import pytest
import torch

from tests.test_transformer_training import run_training, tiny_config
from tests.utils import dist_launcher

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]

ARCH = {"vocab_size": 1024, "hidden_size": 256, "num_layers": 2, "num_attention_heads": 4, "sequence_length": 256,
        "precision": "bfloat16", "relative_position_embedding_type": "rotary"}


def _gpu_config(world_size, **kw):
    dp = world_size // (kw.get("mp", 1) * kw.get("pp", 1))
    kw.setdefault("micro", 4 * dp)  # tiny_config divides by dp: 4 samples per rank and micro batch
    cfg = tiny_config(world_size, arch=dict(ARCH, **kw.pop("arch", {})), **kw)
    cfg["topology"]["device"] = "cuda"
    cfg["topology"]["backend"] = "nccl"
    return cfg


def _run(rank, world_size, port, device, config, env, save_initial=None):
    os.environ.update(env)
    return run_training(rank, world_size, port, device, config, save_initial=save_initial)


def _losses(world_size, env=None, save_initial=None, **kw):
    return dist_launcher(_run, world_size, device="cuda", config=_gpu_config(world_size, **kw), env=env or {},
                         save_initial=save_initial)[0]


def test_fused_zero_matches_nccl(tmp_path: Path):
    """Reduce-scatter / all-gather through peer memory give the losses of the NCCL path (two ranks: the sums have
    one possible order, so the runs agree bit for bit); with and without the multicast mapping."""
    init = str(tmp_path / "init")
    _losses(1, save_initial=init, iters=1)
    nccl = _losses(2, env={"SB200_FUSED_ZERO": "0"}, zero=True, load_dir=init)
    p2p = _losses(2, env={"SB200_FUSED_ZERO": "1", "SB200_P2P_MULTICAST": "0"}, zero=True, load_dir=init)
    mc = _losses(2, env={"SB200_FUSED_ZERO": "1", "SB200_P2P_MULTICAST": "1"}, zero=True, load_dir=init)
    assert nccl[-1] < nccl[0]
    assert p2p == nccl, (p2p, nccl)
    assert mc == nccl, (mc, nccl)


def test_tensor_parallel_matches_single_gpu(tmp_path: Path):
    init = str(tmp_path / "init")
    base = _losses(1, save_initial=init)
    for kw in (dict(mp=2), dict(mp=2, sp=True), dict(pp=2, ga=2, micro=2)):
        got = _losses(2, load_dir=init, **kw)
        for a, b in zip(got, base):
            assert abs(a - b) < 5e-2 * max(1.0, abs(b)), (kw, got, base)


def test_llama_style_tensor_parallel_matches_single_gpu(tmp_path: Path):
    """RMSNorm, SwiGLU, grouped-query attention, interleaved rotary and activation checkpointing under tensor and
    sequence parallelism, with the in-kernel all-reduces forced on for every size."""
    from tests.test_transformer_training import LLAMA_ARCH

    init = str(tmp_path / "init")
    base = _losses(1, save_initial=init, arch=LLAMA_ARCH)
    for kw, env in ((dict(mp=2, ckpt="every_layer"), {"SB200_FUSED_TP": "always"}),
                    (dict(mp=2), {"SB200_FUSED_TP": "0"}), (dict(mp=2, sp=True), {})):
        got = _losses(2, env=env, load_dir=init, arch=LLAMA_ARCH, **kw)
        for a, b in zip(got, base):
            assert abs(a - b) < 5e-2 * max(1.0, abs(b)), (kw, got, base)


def _fused_gemm_allreduce_worker(rank, world_size, port, device):
    import torch.distributed as dist

    from scaling_b200.ops import functional as K
    from scaling_b200.parallel.fused_tp import FusedTPWorkspace

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world_size,
                            device_id=torch.device("cuda", rank))
    dev = torch.device("cuda", rank)
    errors = []
    for multicast in (False, True):
        ws = FusedTPWorkspace(dist.group.WORLD, dev, 4096 * 1024, use_multicast=multicast)
        for M, N, Kd, b_mn in [(256, 256, 128, False), (4096, 768, 384, False), (1000, 264, 200, False),
                               (2048, 768, 1152, True), (128, 64, 64, False)]:
            torch.manual_seed(1 + rank)
            x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
            shape = (Kd, N) if b_mn else (N, Kd)
            w = torch.randn(*shape, device=dev, dtype=torch.bfloat16) * 0.05
            bias = None if b_mn else torch.randn(N, device=dev, dtype=torch.bfloat16)
            ref = K.gemm(x, w, b_mn=b_mn, bias=bias if rank == 0 else None)
            dist.all_reduce(ref)
            got = ws.gemm_allreduce(x, w, bias if rank == 0 else None, b_mn=b_mn)
            again = ws.gemm_allreduce(x, w, bias if rank == 0 else None, b_mn=b_mn)
            torch.cuda.synchronize()
            K.check_status()
            rel = ((got.float() - ref.float()).norm() / ref.float().norm()).item()
            # peer loads add in rank order like the library; the switch's adder rounds once from fp32
            errors.append((multicast and ws.use_multicast, (M, N, Kd, b_mn), rel, torch.equal(got, again)))
        del ws
    return errors


def test_gemm_with_in_kernel_allreduce():
    results = dist_launcher(_fused_gemm_allreduce_worker, 2, device="cuda")
    for per_rank in results:
        for multicast, shape, rel, repeatable in per_rank:
            assert repeatable, shape
            assert rel < (6e-3 if multicast else 1e-6), (multicast, shape, rel)


def _fused_sequence_parallel_worker(rank, world_size, port, device):
    import torch.distributed as dist

    from scaling_b200.ops import functional as K
    from scaling_b200.parallel.fused_tp import FusedTPWorkspace

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world_size,
                            device_id=torch.device("cuda", rank))
    dev = torch.device("cuda", rank)
    results = []
    for multicast in (False, True):
        ws = FusedTPWorkspace(dist.group.WORLD, dev, 4096 * 2048, use_multicast=multicast)
        for M, N, Kd, b_mn in [(256, 256, 128, False), (4096, 768, 384, False), (1024, 264, 200, False),
                               (2048, 1152, 768, True), (512, 64, 64, False)]:
            torch.manual_seed(1 + rank)
            shape = (Kd, N) if b_mn else (N, Kd)
            w = torch.randn(*shape, device=dev, dtype=torch.bfloat16) * 0.05
            bias = None if b_mn else torch.randn(N, device=dev, dtype=torch.bfloat16)
            # reduce-scatter: rows [rank * M / W, ...) of the summed product
            x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
            ref = K.gemm(x, w, b_mn=b_mn, bias=bias if rank == 0 else None)
            dist.all_reduce(ref)
            ref = ref[rank * (M // world_size):(rank + 1) * (M // world_size)]
            got = ws.gemm_reduce_scatter(x, w, bias if rank == 0 else None, b_mn=b_mn)
            again = ws.gemm_reduce_scatter(x, w, bias if rank == 0 else None, b_mn=b_mn)
            torch.cuda.synchronize()
            K.check_status()
            rel = ((got.float() - ref.float()).norm() / ref.float().norm()).item()
            results.append(("rs", multicast and ws.use_multicast, (M, N, Kd, b_mn), rel, torch.equal(got, again)))
            # all-gather: every rank multiplies all ranks' rows
            shard = torch.randn(M // world_size, Kd, device=dev, dtype=torch.bfloat16)
            full = torch.empty(M, Kd, device=dev, dtype=torch.bfloat16)
            dist.all_gather_into_tensor(full, shard)
            act = "none" if b_mn else "gelu"
            pre_ref = torch.empty(M, N, device=dev, dtype=torch.bfloat16) if act == "gelu" else None
            ref = K.gemm(full, w, b_mn=b_mn, bias=bias, act=act, pre_act_out=pre_ref)
            pre = torch.empty_like(pre_ref) if pre_ref is not None else None
            got = ws.allgather_gemm(shard, w, bias, act, pre, b_mn=b_mn)
            torch.cuda.synchronize()
            K.check_status()
            same = torch.equal(got, ref) and torch.equal(ws.gathered(M, Kd), full)
            if pre is not None:
                same = same and torch.equal(pre, pre_ref)
            cached = ws.cached_gather(shard)
            results.append(("ag", multicast and ws.use_multicast, (M, N, Kd, b_mn), 0.0 if same else 1.0,
                            cached is not None and torch.equal(cached, full)))
        del ws
    return results


def test_gemm_with_in_kernel_reduce_scatter_and_all_gather():
    for per_rank in dist_launcher(_fused_sequence_parallel_worker, 2, device="cuda"):
        for kind, multicast, shape, rel, ok in per_rank:
            assert ok, (kind, shape)
            assert rel < (6e-3 if multicast and kind == "rs" else 1e-6), (kind, multicast, shape, rel)
