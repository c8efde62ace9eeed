"""Padding / position helpers (reference: omegalax/models/qwen3/utils.py)."""
from __future__ import annotations

import torch

PAD_POSITION = 2 ** 30


def count_left_pads(segment_ids):
    """Number of leading zeros per row of a [B,T] segment-id tensor."""
    nz = (segment_ids != 0).to(torch.int32)
    return (nz.cumsum(-1) == 0).sum(-1).to(torch.int32)


def count_right_pads(token_ids, pad_id: int) -> int:
    """Largest number of trailing pad tokens over the batch (an all-pad row counts T)."""
    is_pad = token_ids == pad_id
    trailing = torch.flip(is_pad, dims=[-1]).to(torch.int32).cumprod(-1).sum(-1)
    return int(trailing.max().item()) if trailing.numel() else 0


def compute_positions_from_segment_ids(segment_ids):
    """Position = t - index of the first real token for real tokens, 2**30 for padding."""
    B, T = segment_ids.shape
    real = segment_ids != 0
    first = count_left_pads(segment_ids).to(torch.int64)
    t = torch.arange(T, device=segment_ids.device, dtype=torch.int64)[None, :]
    pos = t - first[:, None]
    return torch.where(real, pos, torch.full_like(pos, PAD_POSITION))
