"""Tensor-parallel slices of Qwen3.5 parameters.

The reference maps the logical axes heads / kv_heads / mlp / vocab to the tp mesh axis
(omegalax/models/shard_config.py:11-19).  Here tensor parallelism covers the gated full-attention
layers (heads and kv heads over tp): the fused projection keeps whole heads per rank -- for the
queries a head is its [q | gate] pair of row blocks -- and the output projection keeps the
matching input columns.  GatedDeltaNet layers, the MLP / routed experts, norms, embedding, head
and the vision tower are replicated over tp and work on sequence-parallel rows.
"""
from __future__ import annotations

import torch

from ...parallel import tp as tp_lib


def _text(cfg):
    return getattr(cfg, "text_config", cfg)


def _is_attn(name: str, leaf: str) -> bool:
    return ".attn." in f".{name}" and name.endswith(leaf) and "visual." not in name


def tp_slice(name: str, tensor: torch.Tensor, cfg, tp: int, rank: int) -> torch.Tensor:
    """Slice of a full (tp = 1) parameter that tensor-parallel rank ``rank`` holds."""
    if tp == 1:
        return tensor
    c = _text(cfg)
    if _is_attn(name, "attn.qkv_proj.weight") or _is_attn(name, "attn.qkv_proj.bias"):
        rows = tp_lib.qkv_rows_for_rank(c.num_attention_heads, c.num_key_value_heads, c.head_dim, tp, rank, q_mult=2)
        return tensor[rows]
    if _is_attn(name, "attn.o_proj.weight"):
        return tp_lib.slice_cols(tensor, tp, rank)
    return tensor


def tp_unslice(name: str, parts: list[torch.Tensor], cfg) -> torch.Tensor:
    """Inverse of ``tp_slice``."""
    tp = len(parts)
    if tp == 1:
        return parts[0]
    c = _text(cfg)
    if _is_attn(name, "attn.o_proj.weight"):
        return torch.cat(parts, dim=1)
    if _is_attn(name, "attn.qkv_proj.weight") or _is_attn(name, "attn.qkv_proj.bias"):
        full = torch.empty((sum(p.shape[0] for p in parts), *parts[0].shape[1:]), dtype=parts[0].dtype)
        for r, p in enumerate(parts):
            rows = tp_lib.qkv_rows_for_rank(c.num_attention_heads, c.num_key_value_heads, c.head_dim, tp, r, q_mult=2)
            full[rows] = p
        return full
    return parts[0]
