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


WORLD_SIZES = [2, 4, 8]


def _need(world_size):
    if torch.cuda.device_count() < world_size:
        pytest.skip(f"needs {world_size} GPUs")


def _row_error(got, ref):
    """(relative error of the whole tensor, largest absolute error of a row relative to that row's largest value):
    the second catches a wrong tile edge, a dropped row or swapped columns that a norm over everything would hide."""
    got, ref = got.float(), ref.float()
    rel = ((got - ref).norm() / ref.norm().clamp_min(1e-20)).item()
    row = ((got - ref).abs().amax(dim=-1) / ref.abs().amax(dim=-1).clamp_min(1e-3)).max().item()
    return rel, row


def _init_group(rank, world_size, port):
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world_size,
                            device_id=torch.device("cuda", rank))
    return torch.device("cuda", rank)


def _fused_gemm_allreduce_worker(rank, world_size, port, device):
    import torch.distributed as dist

    from scaling_b200.ops import functional as K
    from scaling_b200.parallel.fused_tp import FusedTPWorkspace

    dev = _init_group(rank, world_size, port)
    W = world_size
    errors = []
    # odd tile counts (tiles not a multiple of the group), N off the 256-wide tile, partial last tile, one tile only
    shapes = [(256, 256, 128, False), (4096, 768, 384, False), (1000, 264, 200, False), (2048, 768, 1152, True),
              (128, 64, 64, False), (128 * (W + 1), 384, 72, False), (128 * W, 640, 256, True), (129, 136, 8, False)]
    for multicast in (False, True):
        ws = FusedTPWorkspace(dist.group.WORLD, dev, 4096 * 1024, use_multicast=multicast)
        for M, N, Kd, b_mn in shapes:
            torch.manual_seed(1 + rank)
            x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
            shape = (Kd, N) if b_mn else (N, Kd)
            w = torch.randn(*shape, device=dev, dtype=torch.bfloat16) * 0.05
            bias = None if b_mn else torch.randn(N, device=dev, dtype=torch.bfloat16)
            ref = K.gemm(x, w, b_mn=b_mn, bias=bias if rank == 0 else None, out_dtype=torch.float32)
            dist.all_reduce(ref)
            got = ws.gemm_allreduce(x, w, bias if rank == 0 else None, b_mn=b_mn)
            again = ws.gemm_allreduce(x, w, bias if rank == 0 else None, b_mn=b_mn)
            torch.cuda.synchronize()
            K.check_status()
            rel, row = _row_error(got, ref)
            errors.append((multicast and ws.use_multicast, (M, N, Kd, b_mn), rel, row, torch.equal(got, again)))
        del ws
    return errors


@pytest.mark.parametrize("world_size", WORLD_SIZES)
def test_gemm_with_in_kernel_allreduce(world_size):
    """Sum over the ranks of x_r w_r^T from one launch per rank against fp32 partial products summed by the library;
    bf16 partial tiles cost one rounding per rank (two with the switch's adder)."""
    _need(world_size)
    results = dist_launcher(_fused_gemm_allreduce_worker, world_size, device="cuda")
    for per_rank in results:
        for multicast, shape, rel, row, repeatable in per_rank:
            assert repeatable, shape
            assert rel < 6e-3 and row < 3e-2, (multicast, shape, rel, row)


def _fused_sequence_parallel_worker(rank, world_size, port, device):
    import torch.distributed as dist

    from scaling_b200.ops import functional as K
    from scaling_b200.parallel.fused_tp import FusedTPWorkspace

    dev = _init_group(rank, world_size, port)
    W = world_size
    results = []
    shapes = [(128 * W, 256, 128, False), (4096, 768, 384, False), (1024 * W // 2, 264, 200, False),
              (2048, 1152, 768, True), (256 * W, 64, 64, False), (384 * W, 640, 72, True)]
    for multicast in (False, True):
        ws = FusedTPWorkspace(dist.group.WORLD, dev, 4096 * 2048, use_multicast=multicast)
        for M, N, Kd, b_mn in shapes:
            torch.manual_seed(1 + rank)
            shape = (Kd, N) if b_mn else (N, Kd)
            w = torch.randn(*shape, device=dev, dtype=torch.bfloat16) * 0.05
            bias = None if b_mn else torch.randn(N, device=dev, dtype=torch.bfloat16)
            # reduce-scatter: rows [rank * M / W, ...) of the summed product
            x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
            ref = K.gemm(x, w, b_mn=b_mn, bias=bias if rank == 0 else None, out_dtype=torch.float32)
            dist.all_reduce(ref)
            ref = ref[rank * (M // W):(rank + 1) * (M // W)]
            got = ws.gemm_reduce_scatter(x, w, bias if rank == 0 else None, b_mn=b_mn)
            again = ws.gemm_reduce_scatter(x, w, bias if rank == 0 else None, b_mn=b_mn)
            torch.cuda.synchronize()
            K.check_status()
            rel, row = _row_error(got, ref)
            results.append(("rs", multicast and ws.use_multicast, (M, N, Kd, b_mn), max(rel, row / 5),
                            torch.equal(got, again)))
            # all-gather: every rank multiplies all ranks' rows (no arithmetic crosses the ranks: exact)
            shard = torch.randn(M // W, Kd, device=dev, dtype=torch.bfloat16)
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
            # a second gather right behind the first: the operand buffers alternate between launches
            shard2 = torch.randn(M // W, Kd, device=dev, dtype=torch.bfloat16)
            full2 = torch.empty(M, Kd, device=dev, dtype=torch.bfloat16)
            dist.all_gather_into_tensor(full2, shard2)
            got2 = ws.allgather_gemm(shard2, w, bias, "none", None, b_mn=b_mn)
            torch.cuda.synchronize()
            K.check_status()
            results.append(("ag2", multicast and ws.use_multicast, (M, N, Kd, b_mn),
                            0.0 if torch.equal(got2, K.gemm(full2, w, b_mn=b_mn, bias=bias)) else 1.0,
                            torch.equal(ws.gathered(M, Kd), full2)))
        del ws
    return results


@pytest.mark.parametrize("world_size", WORLD_SIZES)
def test_gemm_with_in_kernel_reduce_scatter_and_all_gather(world_size):
    _need(world_size)
    for per_rank in dist_launcher(_fused_sequence_parallel_worker, world_size, device="cuda"):
        for kind, multicast, shape, err, ok in per_rank:
            assert ok, (kind, shape)
            assert err < (6e-3 if kind == "rs" else 1e-6), (kind, multicast, shape, err)


@pytest.mark.parametrize("world_size", [4, 8])
def test_llama_style_tensor_parallel_on_larger_groups(tmp_path: Path, world_size):
    """The llama-style model over four and eight tensor-parallel ranks (sequence parallel, fused kernels) against
    one GPU; with eight ranks the two KV heads are replicated within pairs of ranks."""
    _need(world_size)
    from tests.test_transformer_training import LLAMA_ARCH

    arch = dict(LLAMA_ARCH, hidden_size=512, num_attention_heads=8,
                attention_num_kv_heads=2 if world_size == 8 else 4, sequence_length=128 * world_size // 4)
    init = str(tmp_path / "init")
    base = _losses(1, save_initial=init, arch=arch)
    for kw, env in ((dict(mp=world_size, sp=True), {}), (dict(mp=world_size), {"SB200_FUSED_TP": "always"})):
        got = _losses(world_size, env=env, load_dir=init, arch=arch, **kw)
        for a, b in zip(got, base):
            assert abs(a - b) < 5e-2 * max(1.0, abs(b)), (kw, got, base)
