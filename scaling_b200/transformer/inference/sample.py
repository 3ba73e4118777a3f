"""Next-token selection on ``logits[batch, seq, vocab]`` (src/scaling/transformer/inference/sample.py:5-45).

Every ``sample_*`` function returns the chosen id for the last position of each batch row; the ``*_transform``
functions return filtered logits to be passed on to a sampler.
"""

from __future__ import annotations

import torch


def sample_argmax(logits: torch.Tensor) -> torch.Tensor:
    return logits[:, -1].argmax(dim=-1)


def _inverse_cdf_draw(probs: torch.Tensor) -> torch.Tensor:
    """One categorical draw per row by inverting the CDF with a single uniform number (no sync, no sort)."""
    u = torch.rand(probs.shape[:-1], device=probs.device, dtype=probs.dtype).unsqueeze(-1)
    return (probs.cumsum(-1) >= u).to(torch.uint8).argmax(-1)


def sample_temperature(logits: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    probs = torch.softmax(logits[:, -1].float() / temperature, dim=-1)
    return _inverse_cdf_draw(probs)


def top_k_transform(logits: torch.Tensor, k: int = 10) -> torch.Tensor:
    """Keep the ``k`` largest logits of every position, set the rest to -inf."""
    kth = torch.topk(logits, k, dim=-1).values[..., -1:]
    return logits.masked_fill(logits < kth, float("-inf"))


def top_p_transform(logits: torch.Tensor, threshold: float = 0.95) -> torch.Tensor:
    """Nucleus filter: keep the smallest set of tokens whose probability mass exceeds ``threshold``."""
    sorted_logits, order = torch.sort(logits, descending=True, dim=-1)
    mass = torch.softmax(sorted_logits.float(), dim=-1).cumsum(-1)
    drop_sorted = mass > threshold
    # shift right so that the first token crossing the threshold stays in
    drop_sorted = torch.cat((torch.zeros_like(drop_sorted[..., :1]), drop_sorted[..., :-1]), dim=-1)
    drop = torch.zeros_like(drop_sorted).scatter(-1, order, drop_sorted)
    return logits.masked_fill(drop, float("-inf"))
