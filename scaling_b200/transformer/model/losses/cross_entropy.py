"""Token-level cross-entropy, evaluated on vocabulary shards.

``loss = sum(ce_t * w_t) / sum(w_t)`` with fp32 statistics and an accuracy metric over tokens with
positive weight - the reference's loss (src/scaling/transformer/model/losses/cross_entropy.py:12-88).
Under tensor parallelism the logits arrive sharded over the vocabulary: each rank reduces its shard
to (max, sum-exp, target logit, arg-max) per token with one kernel, three tiny all-reduces combine
them, and a second kernel writes loss and d logits for the local shard.  The full ``[tokens, vocab]``
matrix is neither gathered nor copied to fp32.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ....core.nn.scale import scale_bwd, scale_fwd
from ....core.nn.umup import UMuParametrization
from ....ops import functional as K
from ....parallel.topology import Topology
from ...context.config import CrossEntropyLossFunctionConfig, UMuPConfig
from ...data.text_dataset_batch import TextDatasetBatch
from ..layers.base import TransformerLayerIO


class _VocabParallelCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, coef, group, vocab_start, overwrite=False):  # type: ignore[override]
        """logits ``[N, V_local]``, targets ``[N]``, coef ``[N]`` (weight / sum of weights).
        Returns (loss scalar fp32, global arg-max ``[N]``)."""
        rmax, rsum, tgt, aval, aidx = K.ce_stats(logits, targets, vocab_start)
        if group is not None:
            gmax = rmax.clone()
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
            packed = torch.stack((rsum * torch.exp(rmax - gmax), tgt))
            dist.all_reduce(packed, group=group)
            gsum, gtgt = packed[0], packed[1]
            # lowest index among the shards that hold the global maximum
            cand = torch.where(aval >= gmax, aidx, torch.full_like(aidx, torch.iinfo(torch.int64).max))
            dist.all_reduce(cand, op=dist.ReduceOp.MIN, group=group)
            argmax = cand
        else:
            gmax, gsum, gtgt, argmax = rmax, rsum, tgt, aidx
        # The loss needs the row statistics only.  The gradient with respect to the logits is written in the backward
        # pass, already multiplied by the upstream gradient; over the logits themselves when their producer has said
        # that nobody else reads them (``overwrite``: the language-model heads do so in training), so that the
        # [tokens, vocabulary] matrix is read once here and read and written once there.  Logits from anywhere else
        # (a tensor the caller still holds) are left alone and the gradient gets its own buffer.
        loss_tok = torch.log(gsum) + gmax - gtgt
        ctx.save_for_backward(logits, targets, gmax, gsum, gtgt, coef)
        ctx.vocab_start = vocab_start
        ctx.overwrite = bool(overwrite)
        ctx.mark_non_differentiable(argmax)
        return (loss_tok * coef).sum(), argmax

    @staticmethod
    def backward(ctx, grad_loss, _grad_argmax):  # type: ignore[override]
        logits, targets, gmax, gsum, gtgt, coef = ctx.saved_tensors
        _, dlogits = K.ce_finalize(logits, targets, gmax, gsum, gtgt, coef, ctx.vocab_start, want_grad=True,
                                   inplace=logits.is_cuda and ctx.overwrite, scale_dev=grad_loss)
        return dlogits, None, None, None, None, None


def vocab_parallel_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, weights: torch.Tensor,
                                 topology: Optional[Topology], sharded: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """(weighted mean loss, arg-max token id per position)."""
    group = None
    start = 0
    if sharded and topology is not None and topology.config.model_parallel_size > 1:
        group = topology.model_parallel_group
        start = topology.model_parallel_rank * logits.shape[-1]
    w = weights.float().reshape(-1)
    coef = w / w.sum()
    overwrite = bool(getattr(logits, "_sb200_loss_may_overwrite", False)) and logits.is_contiguous()
    flat = logits.reshape(-1, logits.shape[-1])
    return _VocabParallelCrossEntropy.apply(flat, targets.reshape(-1), coef, group, start, overwrite)


class CrossEntropyLoss(torch.nn.Module):
    def __init__(self, loss_config: CrossEntropyLossFunctionConfig, umup_config: UMuPConfig,
                 topology: Optional[Topology] = None, vocab_size: Optional[int] = None):
        super().__init__()
        self._use_umup = umup_config.enable
        self.umup_loss_mult = umup_config.loss_mult
        self.topology = topology
        self.vocab_size = vocab_size

    def forward(self, output: TransformerLayerIO, batch: TextDatasetBatch) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        assert batch.target_token_ids is not None, (
            "target_token_ids not set in batch; you may want to revisit the implementation of Batch.only_targets()"
        )
        assert batch.loss_weights is not None, (
            "loss_weights not set in batch; you may want to revisit the implementation of Batch.only_targets()"
        )
        logits = output.activations
        local_vocab = logits.shape[-1]
        sharded = self.vocab_size is not None and local_vocab != self.vocab_size
        if self._use_umup:
            full_vocab = self.vocab_size or local_vocab
            fwd, bwd = UMuParametrization.get_umup_cross_entropy_scales(self.umup_loss_mult, full_vocab)
            disposable = getattr(logits, "_sb200_loss_may_overwrite", False)
            scaled = scale_bwd(scale_fwd(logits, fwd), bwd)
            if disposable or scaled.data_ptr() != logits.data_ptr():  # the producer's word, or a copy of our own
                scaled._sb200_loss_may_overwrite = True  # type: ignore[attr-defined]
            logits = scaled
        weights = batch.loss_weights.float().reshape(-1)
        targets = batch.target_token_ids.reshape(-1)
        loss, argmax = vocab_parallel_cross_entropy(logits, targets, weights, self.topology, sharded)
        if self._use_umup:
            # Unit scaling: the division by the sum of the loss weights acts on the value of the loss only, the
            # gradient is that of the weighted sum (src/scaling/transformer/model/losses/cross_entropy.py:47-56 scales
            # the summed loss with scale_fwd), so the logits receive gradients of unit scale whatever the batch size.
            loss = scale_bwd(loss, weights.sum())
        mask = (weights > 0).float()
        accuracy = ((argmax == targets).float() * mask).sum() / mask.sum()
        return loss, {"accuracy": accuracy}
