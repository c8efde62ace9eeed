"""Rotary embeddings of Qwen3.5: 2-D rope for the vision tower and interleaved partial
multimodal rope (MRoPE) for the text decoder (reference: omegalax/models/qwen3_5/rope.py)."""
from __future__ import annotations

import torch

from ...ops import reference as R


def apply_vision_rope(x, cos, sin):
    """Rotate-half over the whole head in fp32, cast back.  x [N, heads, K]; cos/sin [N, K]."""
    dt = x.dtype
    xf = x.float()
    c, s = cos.float().unsqueeze(1), sin.float().unsqueeze(1)
    half = xf.shape[-1] // 2
    rot = torch.cat([-xf[..., half:], xf[..., :half]], dim=-1)
    return (xf * c + rot * s).to(dt)


def interleave_mrope(freqs_ZBTF, mrope_section):
    """freqs [3,B,T,F] (temporal, height, width) -> [B,T,F]: slot i takes the height
    position if i in {1,4,7,...} and i < 3*sec[1], the width position if i in {2,5,8,...}
    and i < 3*sec[2], else the temporal position."""
    out = freqs_ZBTF[0].clone()
    for axis, offset in ((1, 1), (2, 2)):
        idx = slice(offset, mrope_section[axis] * 3, 3)
        out[..., idx] = freqs_ZBTF[axis][..., idx]
    return out


def generate_text_rope(position_ids_ZBT, head_dim: int, partial_rotary_factor: float, theta: float,
                       mrope_section):
    """fp32 (cos, sin) of shape [B, T, rotary_dim] with emb = concat(freqs, freqs)."""
    rotary_dim = int(head_dim * partial_rotary_factor)
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32,
                                        device=position_ids_ZBT.device) / rotary_dim))
    freqs = position_ids_ZBT.to(torch.float32)[..., None] * inv  # [3,B,T,F]
    f = interleave_mrope(freqs, mrope_section)
    emb = torch.cat([f, f], dim=-1)
    return torch.cos(emb), torch.sin(emb)


def mrope_half_tables(position_ids_ZBT, rotary_dim: int, theta: float, mrope_section):
    """fp32 (sin, cos) of shape [B, T, rotary_dim/2] -- the form the fused kernel consumes."""
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32,
                                        device=position_ids_ZBT.device) / rotary_dim))
    freqs = position_ids_ZBT.to(torch.float32)[..., None] * inv
    f = interleave_mrope(freqs, mrope_section)
    return torch.sin(f), torch.cos(f)


def apply_text_rope(x, cos, sin):
    """Rotate-half on the first rotary_dim channels of x [B,T,heads,K]; the rest pass through.
    cos/sin [B,T,rotary_dim] are cast to x.dtype before use."""
    rot = cos.shape[-1]
    half = rot // 2
    return R.apply_rope(x, sin[..., :half], cos[..., :half], rot)
