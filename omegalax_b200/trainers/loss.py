"""Next-token cross-entropy over a large vocabulary without materialising [B,T,V] logits.

``chunked_cross_entropy_loss`` shifts (hidden[:, :-1] predicts targets[:, 1:]), walks the
rows in tiles, and returns sum(nll * mask) / max(sum(mask), 1).  On CUDA bf16 each tile is
one tcgen05 GEMM whose epilogue takes the softmax statistics from the fp32 accumulator (the
loss is that of fp32 logits, as in the reference) and writes a bf16 logits tile, an in-place
dlogits kernel, and the two gradient GEMMs, so the backward needs no recomputation (reference
semantics: omegalax/trainers/loss.py:38-116, which tiles along T and rematerialises each tile).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import functional as Fn


def supervised_count(mask_BT, group=None) -> torch.Tensor:
    """Number of supervised target positions (sum of mask[:, 1:]) over all data ranks."""
    n = mask_BT[:, 1:].to(torch.float32).sum().reshape(1)
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(n, group=group)
    return n


def chunked_cross_entropy_loss(hidden_BTD, lm_head_VD, targets_BT, mask_BT, num_tiles: int = 8,
                               *, group=None, count: torch.Tensor | None = None):
    """Masked mean next-token NLL.  ``lm_head_VD`` is the [vocab, hidden] projection weight.
    ``count`` overrides the normaliser (e.g. the global supervised-token count under data
    parallelism, so that the sum of the per-rank losses is the global mean)."""
    B, T, D = hidden_BTD.shape
    # All B*T rows go through the head, with the targets shifted left and the last position of every
    # sequence masked out: slicing hidden[:, :-1] would copy the whole activation (B*(T-1)*D
    # elements) just to drop B rows, whereas the shifted targets and mask are B*T integers.
    h = hidden_BTD.reshape(-1, D)
    tgt = torch.zeros_like(targets_BT)
    tgt[:, :-1] = targets_BT[:, 1:]
    tgt = tgt.reshape(-1)
    mask = torch.zeros(B, T, dtype=torch.float32, device=mask_BT.device)
    mask[:, :-1] = mask_BT[:, 1:].to(torch.float32)
    mask = mask.reshape(-1)
    if count is None:
        count = supervised_count(mask_BT, group)
    scale = 1.0 / count.clamp_min(1.0)
    rows = h.shape[0]
    chunk = max(1, -(-rows // max(num_tiles, 1)))
    if h.is_cuda:
        chunk = min(max(chunk, 1024), 8192)
    return Fn.linear_cross_entropy(h, lm_head_VD, tgt, mask, scale, chunk=chunk)
