"""Tensor-parallel slices of Qwen3 parameters.

Column-parallel projections keep whole heads / whole (gate, up) pairs per rank; row-parallel
projections keep the matching input columns; everything else is replicated over tp.
"""
from __future__ import annotations

import torch

from ...parallel import tp as tp_lib


def tp_slice(name: str, tensor: torch.Tensor, cfg, tp: int, rank: int) -> torch.Tensor:
    """Slice of a full (tp = 1) native parameter that tensor-parallel rank ``rank`` holds."""
    if tp == 1:
        return tensor
    if name.endswith("attn.qkv_proj.weight") or name.endswith("attn.qkv_proj.bias"):
        rows = tp_lib.qkv_rows_for_rank(cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, tp, rank)
        return tensor[rows]
    if name.endswith("attn.o_proj.weight"):
        return tp_lib.slice_cols(tensor, tp, rank)
    if name.endswith("mlp.gate_up_proj.weight"):
        return tensor[tp_lib.gate_up_rows_for_rank(tensor.shape[0] // 2, tp, rank)]
    if name.endswith("mlp.down_proj.weight"):
        return tp_lib.slice_cols(tensor, tp, rank)
    if name == "lm_head.weight" and _vocab_parallel(cfg, tp):
        return tp_lib.slice_rows(tensor, tp, rank)
    return tensor


def _vocab_parallel(cfg, tp: int) -> bool:
    from .model import vocab_parallel_head

    return vocab_parallel_head(cfg, tp)


def tp_unslice(name: str, parts: list[torch.Tensor], cfg) -> torch.Tensor:
    """Inverse of ``tp_slice``: assemble the full parameter from the per-rank slices."""
    tp = len(parts)
    if tp == 1:
        return parts[0]
    if name == "lm_head.weight" and _vocab_parallel(cfg, tp):
        return torch.cat(parts, dim=0)
    if name.endswith("attn.o_proj.weight") or name.endswith("mlp.down_proj.weight"):
        return torch.cat(parts, dim=1)
    if name.endswith("attn.qkv_proj.weight") or name.endswith("attn.qkv_proj.bias"):
        full = torch.empty((sum(p.shape[0] for p in parts), *parts[0].shape[1:]), dtype=parts[0].dtype)
        for r, p in enumerate(parts):
            full[tp_lib.qkv_rows_for_rank(cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, tp, r)] = p
        return full
    if name.endswith("mlp.gate_up_proj.weight"):
        F = sum(p.shape[0] for p in parts) // 2
        full = torch.empty((2 * F, parts[0].shape[1]), dtype=parts[0].dtype)
        for r, p in enumerate(parts):
            full[tp_lib.gate_up_rows_for_rank(F, tp, r)] = p
        return full
    return parts[0]


def shard_model_for_tp(full_model, cfg, tp: int, rank: int, device=None, dtype=None):
    """Build the tensor-parallel model of one rank from a full model."""
    from .model import Qwen3

    out = Qwen3(cfg, device=device, dtype=dtype or next(full_model.parameters()).dtype, tp_size=tp)
    src = dict(full_model.named_parameters())
    with torch.no_grad():
        for n, p in out.named_parameters():
            p.copy_(tp_slice(n, src[n], cfg, tp, rank))
    return out
