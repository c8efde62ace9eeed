"""Tensor-parallel slices of Qwen3.5 parameters.

The reference maps the logical axes heads / kv_heads / mlp / vocab to the tp mesh axis
(omegalax/models/shard_config.py:11-19).  Here:

gated attention   whole heads per rank in the fused projection -- a query head is its [q | gate]
                  pair of row blocks -- and the matching input columns of the output projection
GatedDeltaNet     nk/tp key heads and the nv/tp value heads that read them: rows of the q / k / v
                  blocks of in_proj_qkv and the same channels of the conv filter, rows of z / b / a,
                  entries of dt_bias / A_log, input columns of out_proj
MLP, shared expert  whole (gate, up) pairs per rank, matching input columns of the down projection

Routed experts, router, norms, embedding, head and the vision tower are replicated over tp and
work on sequence-parallel rows.
"""
from __future__ import annotations

import torch

from ...parallel import tp as tp_lib


def _text(cfg):
    return getattr(cfg, "text_config", cfg)


def _leaf(name: str, *leaves: str) -> bool:
    return not name.startswith("visual.") and any(name.endswith(x) for x in leaves)


def _gdn_rows(c, tp: int, rank: int) -> torch.Tensor:
    """Rows of in_proj_qkv (= channels of the conv filter) of one rank: its key heads' q and k
    blocks and its value heads' v block."""
    nk, nv, ak, av = c.linear_num_key_heads, c.linear_num_value_heads, c.linear_key_head_dim, c.linear_value_head_dim
    kd = nk * ak
    q = torch.arange(rank * (nk // tp) * ak, (rank + 1) * (nk // tp) * ak)
    v = torch.arange(rank * (nv // tp) * av, (rank + 1) * (nv // tp) * av)
    return torch.cat([q, kd + q, 2 * kd + v])


_ROWS = ("linear_attn.in_proj_z.weight", "linear_attn.in_proj_b.weight", "linear_attn.in_proj_a.weight",
         "linear_attn.dt_bias", "linear_attn.A_log")
_COLS = ("attn.o_proj.weight", "linear_attn.out_proj.weight", "mlp.down_proj.weight", "shared_expert.down_proj.weight")
_GATE_UP = ("mlp.gate_up_proj.weight", "shared_expert.gate_up_proj.weight")
_GDN_QKV = ("linear_attn.in_proj_qkv.weight", "linear_attn.conv_weight")
_ATTN_QKV = (".attn.qkv_proj.weight", ".attn.qkv_proj.bias")


def _rows_for(name: str, n_rows: int, c, tp: int, rank: int):
    """Row indices (dimension 0) of rank ``rank`` for a row-split parameter, else None."""
    if _leaf(name, *_ATTN_QKV):
        return tp_lib.qkv_rows_for_rank(c.num_attention_heads, c.num_key_value_heads, c.head_dim, tp, rank, q_mult=2)
    if _leaf(name, *_GDN_QKV):
        return _gdn_rows(c, tp, rank)
    if _leaf(name, *_GATE_UP):
        return tp_lib.gate_up_rows_for_rank(n_rows // 2, tp, rank)
    if _leaf(name, *_ROWS):
        per = n_rows // tp
        return torch.arange(rank * per, (rank + 1) * per)
    return None


def tp_slice(name: str, tensor: torch.Tensor, cfg, tp: int, rank: int) -> torch.Tensor:
    """Slice of a full (tp = 1) parameter that tensor-parallel rank ``rank`` holds."""
    if tp == 1:
        return tensor
    c = _text(cfg)
    if _leaf(name, *_COLS):
        return tp_lib.slice_cols(tensor, tp, rank)
    rows = _rows_for(name, tensor.shape[0], c, tp, rank)
    return tensor if rows is None else tensor[rows]


def tp_unslice(name: str, parts: list[torch.Tensor], cfg) -> torch.Tensor:
    """Inverse of ``tp_slice``."""
    tp = len(parts)
    if tp == 1:
        return parts[0]
    c = _text(cfg)
    if _leaf(name, *_COLS):
        return torch.cat(parts, dim=1)
    n_rows = sum(p.shape[0] for p in parts)
    if _rows_for(name, n_rows, c, tp, 0) is None:
        return parts[0]
    full = torch.empty((n_rows, *parts[0].shape[1:]), dtype=parts[0].dtype)
    for r, p in enumerate(parts):
        full[_rows_for(name, n_rows, c, tp, r)] = p
    return full
