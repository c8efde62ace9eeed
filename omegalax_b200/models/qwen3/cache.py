"""Contiguous KV cache for decode (reference: omegalax/models/qwen3/cache.py)."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass
class LayerCache:
    k_cache: torch.Tensor      # [B, S, G, K]
    v_cache: torch.Tensor      # [B, S, G, K]
    start_ind: torch.Tensor    # [B] first real position per row, -1 until the first call
    cur_ind: int               # write cursor shared by the batch
    size: int


Cache = list


def cache_size(token_len: int, generate_steps: int) -> int:
    return 2 ** math.ceil(math.log2(max(token_len + generate_steps, 1)))


def init_cache(cfg, batch_size: int, token_len: int, generate_steps: int,
               dtype=torch.bfloat16, device=None) -> Cache:
    S = cache_size(token_len, generate_steps)
    out = []
    for _ in range(cfg.num_layers):
        out.append(LayerCache(
            k_cache=torch.zeros(batch_size, S, cfg.num_kv_heads, cfg.head_dim, dtype=dtype, device=device),
            v_cache=torch.zeros(batch_size, S, cfg.num_kv_heads, cfg.head_dim, dtype=dtype, device=device),
            start_ind=torch.full((batch_size,), -1, dtype=torch.int32, device=device),
            cur_ind=0, size=S))
    return out
