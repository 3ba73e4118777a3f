"""Derived fields of a packed text batch.

``get_cumulative_seq_lengths``: flat cumulative document lengths over the ``b * s`` tokens of a
batch - a boundary after every end-of-document token (id 0) and at every row end (or only at row
ends without attention reset).  ``get_position_ids``: positions restarting after every EOD token.
Padding of the cumulative lengths to the fixed size ``b * (s + 1)`` with -1 keeps pipe-communication
shapes static (src/scaling/transformer/data/utils.py:4-108).  Everything is vectorised; the
reference computes position ids with nested Python loops.
"""

from __future__ import annotations

import torch

EOD_TOKEN = 0


def add_cumulative_seq_lengths_padding(cumulative_seq_lengths: torch.Tensor, pad_to: int,
                                       padding_value: int = -1) -> torch.Tensor:
    assert pad_to >= len(cumulative_seq_lengths)
    pad = torch.full((pad_to - len(cumulative_seq_lengths),), padding_value, dtype=torch.int32,
                     device=cumulative_seq_lengths.device)
    return torch.cat((cumulative_seq_lengths.to(torch.int32), pad))


def remove_cumulative_seq_lengths_padding(cumulative_seq_lengths: torch.Tensor, padding_value: int = -1) -> torch.Tensor:
    return cumulative_seq_lengths[cumulative_seq_lengths != padding_value]


def _document_ends(input_token_ids: torch.Tensor, eod_token: int) -> torch.Tensor:
    """Boolean ``[b, s]``: True at the last token of every document (EOD tokens and row ends)."""
    ends = input_token_ids == eod_token
    ends[:, -1] = True
    return ends


def get_cumulative_seq_lengths(input_token_ids: torch.Tensor, reset_attention_mask: bool = True,
                               eod_token: int = EOD_TOKEN) -> torch.Tensor:
    b, s = input_token_ids.shape
    dev = input_token_ids.device
    if not reset_attention_mask:
        return torch.arange(0, b * s + 1, s, dtype=torch.int32, device=dev)
    flat_ends = _document_ends(input_token_ids, eod_token).reshape(-1).nonzero(as_tuple=True)[0] + 1
    return torch.cat((torch.zeros(1, dtype=torch.int32, device=dev), flat_ends.to(torch.int32)))


def get_cumulative_seq_lengths_padded(input_token_ids: torch.Tensor, reset_attention_mask: bool = True,
                                      eod_token: int = EOD_TOKEN) -> torch.Tensor:
    """Cumulative document lengths padded with -1 to the fixed length ``b * (s + 1)``.

    Computed with fixed-shape operations only (a sort instead of ``nonzero``), so it neither synchronises the
    host nor breaks CUDA-graph capture; equals ``add_cumulative_seq_lengths_padding(get_cumulative_seq_lengths(..))``.
    """
    b, s = input_token_ids.shape
    dev = input_token_ids.device
    total = b * s
    if reset_attention_mask:
        ends = _document_ends(input_token_ids, eod_token).reshape(-1)
    else:
        ends = torch.zeros(b, s, dtype=torch.bool, device=dev)
        ends[:, -1] = True
        ends = ends.reshape(-1)
    big = total + 1
    marks = torch.where(ends, torch.arange(1, total + 1, dtype=torch.int32, device=dev),
                        torch.full((total,), big, dtype=torch.int32, device=dev))
    ordered = torch.sort(marks).values
    ordered = torch.where(ordered == big, torch.full_like(ordered, -1), ordered)
    head = torch.zeros(1, dtype=torch.int32, device=dev)
    tail = torch.full((b - 1,), -1, dtype=torch.int32, device=dev)
    return torch.cat((head, ordered, tail))


def document_ranges_from_padded(cumulative_seq_lengths_padded: torch.Tensor, total: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Per token ``(first token of its document, one past its last token)`` as int32, fixed-shape operations only."""
    cu = cumulative_seq_lengths_padded.to(torch.int64)
    cu = torch.where(cu < 0, torch.full_like(cu, total + 1), cu)
    idx = torch.arange(total, device=cu.device)
    doc = (torch.searchsorted(cu, idx, right=True) - 1).clamp_(0, cu.numel() - 2)
    return cu[doc].to(torch.int32).contiguous(), cu[doc + 1].clamp(max=total).to(torch.int32).contiguous()


def get_position_ids(input_token_ids: torch.Tensor, reset_position_ids: bool = True,
                     eod_token: int = EOD_TOKEN) -> torch.Tensor:
    b, s = input_token_ids.shape
    dev = input_token_ids.device
    idx = torch.arange(s, dtype=torch.long, device=dev).unsqueeze(0).expand(b, s)
    if not reset_position_ids:
        return idx.contiguous()
    ends = _document_ends(input_token_ids, eod_token)
    # start index of the document each token belongs to = 1 + index of the previous document end
    start_marks = torch.zeros(b, s, dtype=torch.long, device=dev)
    start_marks[:, 1:] = torch.where(ends[:, :-1], idx[:, 1:], torch.zeros_like(idx[:, 1:]))
    doc_start = torch.cummax(start_marks, dim=1).values
    return idx - doc_start
