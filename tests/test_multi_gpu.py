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
    cfg = tiny_config(world_size, arch=ARCH, **kw)
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
