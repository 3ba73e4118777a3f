"""Unit-scaled maximal-update parametrisation (u-muP) rules.

Per weight type the (forward, backward, gradient, learning-rate) multipliers, residual/skip
scales and the activation / attention / cross-entropy scale factors.  The numbers reproduce the
reference implementation (src/scaling/core/nn/umup.py:14-216): norm/bias ``(1, 1, B^-1/2, 1)``,
embedding ``(1, 1, (B/V)^-1/2, h^-1/2)``, input ``(n_in^-1/2, n_in^-1/2, B^-1/2, 1)``, hidden
``(.., .., .., n_in^-1/2)``, output ``(1/n_in, n_out^-1/2, B^-1/2, 1)``; learning rates on residual
branches are additionally scaled by ``depth^-1/2`` and weights are re-drawn from N(0, 1).
"""

from __future__ import annotations

import math

import torch

from .parameter_meta import UMUP_WEIGHT_TYPE, CoreParameterMeta, UMuPParameterMeta


def _log_interp(alpha: float, lower: float, upper: float) -> float:
    return math.exp(alpha * math.log(upper) + (1.0 - alpha) * math.log(lower))


class UMuParametrization:
    @staticmethod
    def get_depth_scale(depth: int) -> float:
        return depth ** -0.5

    @staticmethod
    def _fan(meta: CoreParameterMeta, mp: int) -> tuple[int, int]:
        n_out, n_in = meta.local_shape[0], meta.local_shape[1]
        if meta.is_model_parallel and meta.model_parallel_dimension == 1:
            n_in *= mp
        elif meta.is_model_parallel and meta.model_parallel_dimension == 0:
            n_out *= mp
        return n_in, n_out

    @staticmethod
    def get_parameter_multipliers(parameter_meta: CoreParameterMeta, model_parallel_size: int,
                                  effective_batch_size: int, depth: int) -> tuple[float, float, float, float]:
        um = parameter_meta.umup_meta
        assert isinstance(um, UMuPParameterMeta)
        batch = effective_batch_size ** -0.5
        kind = um.weight_type
        if kind in (UMUP_WEIGHT_TYPE.NORM, UMUP_WEIGHT_TYPE.BIAS):
            mult = (1.0, 1.0, batch, 1.0)
        elif kind == UMUP_WEIGHT_TYPE.INPUT_EMBEDDING:
            vocab, hidden = parameter_meta.local_shape[0], parameter_meta.local_shape[1]
            if parameter_meta.is_model_parallel:
                vocab *= model_parallel_size
            mult = (1.0, 1.0, (effective_batch_size / vocab) ** -0.5, hidden ** -0.5)
        else:
            n_in, n_out = UMuParametrization._fan(parameter_meta, model_parallel_size)
            if kind == UMUP_WEIGHT_TYPE.INPUT_WEIGHT:
                mult = (n_in ** -0.5, n_in ** -0.5, batch, 1.0)
            elif kind == UMUP_WEIGHT_TYPE.HIDDEN_WEIGHT:
                mult = (n_in ** -0.5, n_in ** -0.5, batch, n_in ** -0.5)
            elif kind == UMUP_WEIGHT_TYPE.OUTPUT_WEIGHT:
                mult = (1.0 / n_in, n_out ** -0.5, batch, 1.0)
            else:
                raise ValueError(f"unknown u-muP weight type {kind}")
        fwd, bwd, grad, lr = mult
        if um.on_residual:
            lr *= UMuParametrization.get_depth_scale(depth)
        return fwd, bwd, grad, lr

    @staticmethod
    def apply_umup_to_weight(weight: torch.Tensor, model_parallel_size: int, effective_batch_size: int, depth: int,
                             reinitialize: bool = True) -> None:
        meta = weight.core_parameter_meta  # type: ignore[attr-defined]
        um = meta.umup_meta
        assert isinstance(um, UMuPParameterMeta)
        um.forward_multiplier, um.backward_multiplier, um.grad_multiplier, um.lr_multiplier = (
            UMuParametrization.get_parameter_multipliers(meta, model_parallel_size, effective_batch_size, depth)
        )
        meta.scale_lr_gain(um.lr_multiplier)
        if reinitialize:
            with torch.no_grad():
                if um.weight_type == UMUP_WEIGHT_TYPE.NORM:
                    weight.fill_(1.0)
                elif um.weight_type == UMUP_WEIGHT_TYPE.BIAS:
                    weight.zero_()
                else:
                    weight.normal_()

    @staticmethod
    def get_umup_residual_scales(residual_mults: list[float], residual_layer_index: int, pre_norm: bool,
                                 depth: int) -> tuple[float, float]:
        d = UMuParametrization.get_depth_scale(depth)
        variances = [(r * d) ** 2 for r in residual_mults]
        tau = variances[residual_layer_index]
        if pre_norm:
            tau = tau / (1.0 + sum(variances[:residual_layer_index]))
        return (tau / (tau + 1.0)) ** 0.5, (1.0 / (tau + 1.0)) ** 0.5

    @staticmethod
    def get_umup_transformer_residual_mults(residual_mult: float, residual_attn_ratio: float,
                                            num_layers: int) -> list[float]:
        mlp = residual_mult * (2.0 / (1.0 + residual_attn_ratio ** 2)) ** 0.5
        return [residual_attn_ratio * mlp, mlp] * num_layers

    @staticmethod
    def get_umup_gelu_scales(gelu_mult: float) -> float:
        return _log_interp(1.0 / (1.0 + 0.25 / gelu_mult ** 2), 2.0, (2.0 / (1.0 - 1.0 / math.pi)) ** 0.5)

    @staticmethod
    def get_umup_swiglu_scales(swiglu_mult: float) -> float:
        return 1.0 / _log_interp(1.0 / (1.0 + 1.0 / swiglu_mult ** 2), 0.5, 2.0 ** -0.5)

    @staticmethod
    def get_umup_attention_scales(head_dim: int, sequence_length: int, mult: float,
                                  dropout_p: float) -> tuple[float, float]:
        out = (1.0 - dropout_p) ** 0.5
        out /= _log_interp(1.0 / (1.0 + 4.0 * head_dim / mult ** 2),
                           math.sqrt(math.log(sequence_length) / sequence_length), 1.0)
        return mult / head_dim, out

    @staticmethod
    def get_umup_cross_entropy_scales(mult: float, vocab_size: int) -> tuple[float, float]:
        return mult, vocab_size / (vocab_size - 1) ** 0.5
