"""In-batch contrastive loss for embedding fine-tuning.

A batch holds groups of ``[query, positive, hard negative * k]`` pooled embeddings.  Embeddings are
gathered over data-parallel ranks (the local block keeps its autograd graph), cosine scores between
all queries and all passages are scaled and fed to a cross-entropy whose target is each query's own
positive; retrieval metrics (top-k accuracy, mean average precision, cosine statistics) are computed
vectorised on the device.  Semantics of src/scaling/transformer/model/losses/contrastive.py:11-205.
"""

from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ....parallel.topology import Topology
from ...context.config import ContrastiveLossFunctionConfig
from ...data.text_dataset_batch import TextDatasetBatch
from ..layers.base import TransformerLayerIO


class ContrastiveLoss(torch.nn.Module):
    def __init__(self, topology: Topology, loss_config: ContrastiveLossFunctionConfig):
        super().__init__()
        self.nr_hard_negatives = loss_config.number_of_hard_negatives
        self.nr_passages = self.nr_hard_negatives + 1
        self.nr_samples_per_batch = self.nr_hard_negatives + 2
        self.log_verbose_metrics = loss_config.log_verbose_metrics
        self.scale = loss_config.scale
        self.topology = topology

    def _gather(self, t: torch.Tensor) -> torch.Tensor:
        topo = self.topology
        if topo is None or topo.config.data_parallel_size == 1:
            return t
        t = t.contiguous()
        parts = [torch.empty_like(t) for _ in range(topo.config.data_parallel_size)]
        dist.all_gather(parts, t, group=topo.data_parallel_group)
        parts[topo.data_parallel_rank] = t  # keep the graph of the local block
        return torch.cat(parts, dim=0)

    def _split_queries_passages(self, activations: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        group = self.nr_samples_per_batch
        idx = torch.arange(activations.shape[0], device=activations.device)
        is_query = idx % group == 0
        return activations[is_query], activations[~is_query]

    @staticmethod
    def _cos_sim(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        return F.normalize(a, p=2, dim=1) @ F.normalize(b, p=2, dim=1).t()

    def forward(self, output: TransformerLayerIO, batch: TextDatasetBatch) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        activations = self._gather(output.activations)
        queries, passages = self._split_queries_passages(activations)
        scores = self._cos_sim(queries, passages) * self.scale
        target = torch.arange(scores.size(0), device=scores.device, dtype=torch.long) * self.nr_passages
        loss = F.cross_entropy(scores, target)
        metrics = self._compute_metrics(scores.detach(), target) if self.log_verbose_metrics else {}
        return loss, metrics

    def _compute_metrics(self, scores: torch.Tensor, target: torch.Tensor) -> dict[str, torch.Tensor]:
        n, p = scores.shape
        rows = torch.arange(n, device=scores.device)
        positive = scores[rows, target]
        k = self.nr_hard_negatives
        hard = (scores[rows[:, None], target[:, None] + 1 + torch.arange(k, device=scores.device)[None, :]]
                if k > 0 else scores.new_zeros(n, 0))
        others = p - 1 - k
        neg = (scores.sum(1) - positive - hard.sum(1)) / max(others, 1)
        neg_abs = (scores.abs().sum(1) - positive - hard.sum(1)) / max(others, 1)
        rank = (scores > positive[:, None]).sum(1)  # 0 = the positive is ranked first
        metrics = {
            "average_cosine": scores.mean(),
            "average_target_cosine_similarity": positive.mean(),
            "average_in_batch_negative_cosine": neg.mean(),
            "average_absolute_in_batch_negative_cosine": neg_abs.mean(),
        }
        for top in (1, 5, 10):
            if top > 1 and self.nr_samples_per_batch < top:
                continue
            hit = (rank < top).float()
            metrics[f"top_{top}_acc"] = hit.mean()
            metrics[f"top_{top}_map"] = (hit / (rank.float() + 1.0)).mean()
        if k > 0:
            metrics["positive_hard_negative_delta"] = (positive[:, None] - hard).abs().mean()
            metrics["average_hard_negative_cosine_similarity"] = hard.mean()
        return metrics
