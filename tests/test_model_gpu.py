"""Whole-model training on one GPU (bf16, the CUDA kernels) against the same model in fp32 on the CPU (plain PyTorch
operators): the losses of a few optimiser steps from a shared initial checkpoint."""

from pathlib import Path

import pytest
import torch

from tests.test_transformer_training import LLAMA_ARCH, run_training, tiny_config
from tests.utils import dist_launcher

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")]

SIZE = {"vocab_size": 1024, "hidden_size": 256, "num_layers": 2, "num_attention_heads": 4, "sequence_length": 256}
GPT_ARCH = {"relative_position_embedding_type": "rotary"}
WINDOW_ARCH = dict(LLAMA_ARCH, local_attention_window_size=64, attention_num_kv_heads=4)


def _config(device, arch, **kw):
    precision = "bfloat16" if device == "cuda" else "float32"
    cfg = tiny_config(1, arch=dict(SIZE, precision=precision, **arch), iters=4, **kw)
    if device == "cuda":
        cfg["topology"]["device"] = "cuda"
        cfg["topology"]["backend"] = "nccl"
    return cfg


def _losses(device, arch, save_initial=None, **kw):
    return dist_launcher(run_training, 1, device=device, config=_config(device, arch, **kw), save_initial=save_initial)[0]


@pytest.mark.parametrize("name,arch,kw", [
    ("gpt", GPT_ARCH, {}),
    ("llama", LLAMA_ARCH, {}),
    ("llama_checkpointed", LLAMA_ARCH, {"ckpt": "every_layer"}),
    ("sliding_window", WINDOW_ARCH, {}),
])
def test_gpu_training_follows_the_fp32_reference(tmp_path: Path, name, arch, kw):
    init = str(tmp_path / "init")
    gpu = _losses("cuda", arch, save_initial=init, **kw)  # bf16 weights: exactly representable in the fp32 model
    cpu = _losses("cpu", arch, load_dir=init)
    assert len(gpu) == len(cpu) == 4
    for a, b in zip(gpu, cpu):
        assert abs(a - b) < 3e-2 * max(1.0, abs(b)), (name, gpu, cpu)
