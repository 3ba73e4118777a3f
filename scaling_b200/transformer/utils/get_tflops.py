"""Throughput metrics: four FLOP-counting models and PaLM-style model-FLOPs utilisation.

The four estimates reproduce the numbers the reference logs as ``runtime/tflops_{aleph_alpha, electra,
bloom, megatron}`` (src/scaling/transformer/utils/get_tflops.py:12-334): per-token operation tables for
one transformer layer (matmuls as 2*m*n, plus norm / softmax / dropout / rotary / GELU elementwise
costs), times tokens and layers, plus the LM head, times 3 (or 2) for forward + backward.  MFU follows
PaLM: tokens/s divided by ``peak / (6 N + 12 L h s)``.  The peak table includes the B200 (dense bf16;
a measured value from ``MEASURED_PEAKS.json`` is preferred when that file is present), which the
reference lacks - it divides by zero on unknown GPUs.
"""

from __future__ import annotations

import json
from enum import Enum
from pathlib import Path
from typing import Any, Optional

import torch

from ...parallel.topology_config import ActivationCheckpointingType
from ..context.config import TransformerArchitectureConfig


def _layer_flops_per_token(a: TransformerArchitectureConfig, rotary_flops: int) -> int:
    h, s, nh = a.hidden_size, a.sequence_length, a.num_attention_heads
    gelu, softmax, dropout, norm = 8, 5, 4, 5
    terms = [
        norm,                      # input layer norm
        3 * 2 * h * h, 3 * h,      # QKV matmul + bias
        2 * h * s,                 # scores
        softmax * s * nh,
        rotary_flops * h,
        dropout * s * nh,          # dropout on probabilities
        s * nh,                    # score scaling
        2 * s * h,                 # weighted values
        2 * h * h, h,              # dense + bias
        dropout * h, h,            # dropout, residual
        norm,                      # post-attention norm
        2 * h * h * 4, 4 * h,      # MLP in + bias
        gelu * 4 * h,
        2 * h * h * 4, h,          # MLP out + bias
        dropout * h, h,            # dropout, residual
    ]
    return sum(terms)


def _table_tflops(iter_time_s: float, topology: Any, a: TransformerArchitectureConfig, rotary_flops: int,
                  dense_embedding: bool, backward_factor: int) -> float:
    tokens = topology.config.global_batch_size * a.sequence_length
    layers = a.num_layers * tokens * _layer_flops_per_token(a, rotary_flops)
    lm_head = 2 * tokens * a.hidden_size * a.vocab_size
    embedding = lm_head if dense_embedding else 0
    final_norm = 5
    total = backward_factor * (embedding + layers + final_norm + lm_head)
    return total / (iter_time_s * topology.config.world_size * 1e12)


def get_tflops_aleph_alpha(iter_time_s: float, topology: Any, transformer_architecture: TransformerArchitectureConfig) -> float:
    """Electra-style table; sparse embedding lookup; backward counted as twice the forward."""
    return _table_tflops(iter_time_s, topology, transformer_architecture, rotary_flops=6, dense_embedding=False,
                         backward_factor=3)


def get_tflops_electra(iter_time_s: float, topology: Any, transformer_architecture: TransformerArchitectureConfig) -> float:
    """Electra's own convention: dense embedding matmul, backward counted like the forward."""
    return _table_tflops(iter_time_s, topology, transformer_architecture, rotary_flops=4, dense_embedding=True,
                         backward_factor=2)


def get_tflops_bloom(iter_time_s: float, topology: Any, transformer_architecture: TransformerArchitectureConfig) -> float:
    """Megatron-LM paper appendix: ``24 B s l h^2`` and ``4 B s^2 h l`` per pass, 3 passes (4 with recomputation)."""
    a = transformer_architecture
    f = 3 if topology.config.activation_checkpointing_type == ActivationCheckpointingType.DISABLED else 4
    B, s, h, l, V = topology.config.global_batch_size, a.sequence_length, a.hidden_size, a.num_layers, a.vocab_size
    total = 24 * f * B * s * l * h * h + 4 * f * B * s * s * h * l + (2 + f) * B * s * h * V
    return total / (iter_time_s * topology.config.world_size * 1e12)


def get_tflops_megatron(parameter_count: int, iter_time_s: float, topology: Any,
                        transformer_architecture: TransformerArchitectureConfig) -> float:
    a = transformer_architecture
    B, s = topology.config.global_batch_size, a.sequence_length
    ff = B * s * parameter_count * 2 * 3
    attn = B * s * s * a.hidden_size * a.num_layers * 60
    return (ff + attn) / (iter_time_s * topology.config.world_size * 1e12)


class HardwareType(Enum):
    A100 = "a100"
    H100 = "h100"
    H200 = "h200"
    B200 = "b200"
    RTX3090 = "rtx3090"
    RTX4090 = "rtx4090"
    DEFAULT = "default"

    @property
    def max_tflops(self) -> float:
        """Dense bf16/fp16 tensor-core peak in FLOP/s."""
        return {"a100": 312e12, "h100": 989.4e12, "h200": 989.4e12, "b200": 2250e12, "rtx3090": 35.58e12,
                "rtx4090": 82.58e12, "default": 0.0}[self.value]

    @classmethod
    def get_via_torch(cls) -> "HardwareType":
        try:  # ask for the name first: without a device the call itself fails
            name = torch.cuda.get_device_name().replace(" ", "").lower().replace("nvidia", "")
        except Exception:  # noqa: BLE001
            return cls.DEFAULT
        return next((x for x in cls if x != cls.DEFAULT and x.value in name), cls.DEFAULT)


def measured_peak_flops(path: Optional[Path] = None) -> Optional[float]:
    """Sustained bf16 matmul throughput recorded for this machine, if a peaks file is present."""
    for cand in ([path] if path else []) + [Path.cwd() / "MEASURED_PEAKS.json",
                                            Path(__file__).resolve().parents[3] / "MEASURED_PEAKS.json"]:
        try:
            data = json.loads(Path(cand).read_text())
            return float(data.get("bf16_tflops_sustained") or data["bf16_tflops"]) * 1e12
        except Exception:
            continue
    return None


def get_model_flop_utilization_palm(iter_time_s: float, parameter_count: int, topology: Any,
                                    transformer_architecture: TransformerArchitectureConfig,
                                    peak_flops: Optional[float] = None) -> float:
    a = transformer_architecture
    peak = peak_flops if peak_flops is not None else HardwareType.get_via_torch().max_tflops
    if peak <= 0.0:
        return 0.0  # unknown hardware: report no utilisation instead of failing the step
    tokens_per_second = topology.config.global_batch_size * a.sequence_length / iter_time_s
    model_flops = 6 * parameter_count + 12 * a.num_layers * a.hidden_size * a.sequence_length
    return tokens_per_second / (peak * topology.config.world_size / model_flops)


def get_tokens_per_second(iter_time_s: float, topology: Any, transformer_architecture: TransformerArchitectureConfig) -> float:
    return topology.config.global_batch_size * transformer_architecture.sequence_length / iter_time_s
