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


UMUP_ARCH = {"umup": {"enable": True}, "norm_type": "rms", "mlp_bias": False, "attention_bias": False,
             "relative_position_embedding_type": "rotary"}
PEFT_ARCH = dict(GPT_ARCH, bitfit_bias_config={"name": "ft"}, softprompt_config={"name": "sp", "n_tokens": 4},
                 adapter_config={"name": "ad", "attention_downsampling_factor": 0.25, "mlp_downsampling_factor": 0.25},
                 lora_config={"name": "lora", "rank": 4, "alpha": 8, "parallel_modules": ["query", "key", "value", "dense"]})
PEFT_KW = {"groups": [{"group_name": "new", "parameters_include": ["bias_ft", "adapter_ad", "softprompt_sp", "lora"],
                       "weight_decay": 0.0,
                       "learning_rate_scheduler": {"learning_rate": 1e-3, "learning_rate_decay_style": "constant"}}],
           "training": {"allow_missing_params_in_optimizer": True}}


@pytest.mark.parametrize("name,arch,kw", [
    ("gpt", GPT_ARCH, {}),
    ("llama", LLAMA_ARCH, {}),
    ("llama_checkpointed", LLAMA_ARCH, {"ckpt": "every_layer"}),
    ("sliding_window", WINDOW_ARCH, {}),
    ("unit_scaled", UMUP_ARCH, {}),
    ("tied_head", dict(GPT_ARCH, weight_tying=True), {}),
    ("bitfit_adapter_softprompt_lora", PEFT_ARCH, PEFT_KW),
])
def test_gpu_training_follows_the_fp32_reference(tmp_path: Path, name, arch, kw):
    init = str(tmp_path / "init")
    gpu = _losses("cuda", arch, save_initial=init, **kw)  # bf16 weights: exactly representable in the fp32 model
    cpu = _losses("cpu", arch, load_dir=init, **{k: v for k, v in kw.items() if k != "ckpt"})
    assert len(gpu) == len(cpu) == 4
    for a, b in zip(gpu, cpu):
        assert abs(a - b) < 3e-2 * max(1.0, abs(b)), (name, gpu, cpu)


# ---------------------------------------------------------------------------------------------- inference on the GPU
def _inference_module(arch: dict, device: str):
    from scaling_b200.transformer.context.config import TransformerArchitectureConfig
    from scaling_b200.transformer.inference import TransformerInferenceModule
    from scaling_b200.transformer.model.model import get_transformer_layer_specs

    torch.manual_seed(0)
    cfg = TransformerArchitectureConfig.from_dict(arch)
    return TransformerInferenceModule(get_transformer_layer_specs(architecture_config=cfg), devices=(device,))


@pytest.mark.parametrize("name,extra", [("gpt", GPT_ARCH), ("llama", LLAMA_ARCH)])
def test_gpu_inference_matches_the_fp32_module_and_the_cache_agrees_with_recompute(name, extra):
    base = dict(SIZE, weight_tying=False, dropout_embedding=0.0, **extra)
    gpu = _inference_module(dict(base, precision="bfloat16", masked_softmax={"kernel": "flash_attention"}), "cuda:0")
    cpu = _inference_module(dict(base, precision="float32", masked_softmax={"kernel": "torch"}), "cpu")
    # same weights: the fp32 module takes the bf16 values
    state = {k: v.detach().float().cpu() for k, v in gpu.state_dict().items()}
    missing, unexpected = cpu.load_state_dict(state, strict=False)
    assert not unexpected and not [m for m in missing if "inv_freq" not in m and "cache" not in m], (missing, unexpected)
    prompt = [3, 700, 15, 9, 420, 77, 5, 1000, 31, 8]
    lg, lc = gpu.logits(input_tokens=prompt).float().cpu(), cpu.logits(input_tokens=prompt)
    assert lg.shape == lc.shape == (len(prompt), SIZE["vocab_size"])
    assert (lg - lc).abs().max() < 0.15 * max(1.0, lc.abs().max().item()), (lg - lc).abs().max()
    cached = gpu.generate(max_tokens=8, input_tokens=prompt, use_cache=True, stop_tokens=[1023])
    plain = gpu.generate(max_tokens=8, input_tokens=prompt, use_cache=False, stop_tokens=[1023])
    n = min(len(cached.completion_tokens), len(plain.completion_tokens))
    assert n >= 1
    # bf16 rounding may flip a near-tie: compare the logits of the steps up to the first differing token
    same = next((i for i in range(n) if cached.completion_tokens[i] != plain.completion_tokens[i]), n - 1)
    assert torch.allclose(cached.completion_logits[:same + 1].float(), plain.completion_logits[:same + 1].float(),
                          atol=0.1, rtol=0.05)
