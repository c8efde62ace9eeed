"""Rotary embeddings for Qwen3 (reference: omegalax/models/qwen3/rope.py)."""
from __future__ import annotations

from ...ops import reference as R


def generate_pos_embeddings(positions, head_dim: int, rope_theta: float = 1_000_000):
    """fp32 (sin, cos), each positions.shape + (head_dim/2,)."""
    return R.rope_tables(positions, head_dim, rope_theta)


def apply_rope(x, sin, cos):
    """Half-split rotation of x [..., heads, head_dim] in x.dtype."""
    return R.apply_rope(x, sin, cos)
