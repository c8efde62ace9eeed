"""Per-token key ranges for packed / left-padded attention masks.

``segment_ids_to_kstart`` and ``cu_seqlens_to_kstart`` turn segment ids or cumulative sequence
lengths into, for every token, the index of the first key of its own segment (``k_start``);
together with causal masking this gives block-diagonal attention over packed sequences
(reference: omegalax/attention.py:7-45; the PyTorch attention definition in
``ops/reference.py`` consumes ``k_start`` / ``k_end`` directly).
"""
from __future__ import annotations

import torch


def segment_ids_to_kstart(segment_ids_BT: torch.Tensor) -> torch.Tensor:
    """First index of the run of equal segment ids that each token belongs to."""
    B, T = segment_ids_BT.shape
    idx = torch.arange(T, device=segment_ids_BT.device).expand(B, T)
    boundary = torch.ones(B, T, dtype=torch.bool, device=segment_ids_BT.device)
    boundary[:, 1:] = segment_ids_BT[:, 1:] != segment_ids_BT[:, :-1]
    starts = torch.where(boundary, idx, torch.zeros_like(idx))
    return torch.cummax(starts, dim=1).values.to(torch.int32)


def cu_seqlens_to_kstart(cu_seqlens: torch.Tensor, total_tokens: int) -> torch.Tensor:
    """For packed rows: start offset of the sequence that contains each row."""
    rows = torch.arange(total_tokens, device=cu_seqlens.device)
    seg = torch.searchsorted(cu_seqlens[1:].contiguous(), rows, right=True)
    return cu_seqlens[seg].to(torch.int32)
