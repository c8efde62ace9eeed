"""Vision transformer shared by Qwen3.5 and Qwen3-VL.

Input is a packed list of flattened patches [N, C*tp*p*p] (already in merge-block order, as
the HF image processor emits them) with ``grid_thw`` [(t, h, w)] per image.  Stages: patch
projection, bilinearly interpolated learned position embedding on a sqrt(npos) grid, 2-D
rotary (row | col), ``depth`` blocks of LayerNorm -> block-diagonal (per frame) non-causal
attention -> LayerNorm -> MLP, then the 2x2 patch merger.  Qwen3-VL additionally taps
DeepStack features after selected blocks through mergers that normalise *after* the 2x2
shuffle.  References: omegalax/models/qwen3_5/vision.py, omegalax/models/qwen3_vl/vision.py.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import functional as Fn
from ..ops import reference as R
from .qwen3.model import Linear
from .qwen3_5.norms import LayerNorm
from .qwen3_5.rope import apply_vision_rope


from ..utils.profiling import scoped


def token_spatial_coords(grid_thw, merge: int, device=None):
    """(row, col, image_id) of every patch token in merge-block order."""
    rows, cols, img = [], [], []
    for i, (t, h, w) in enumerate(grid_thw):
        mh, mw = h // merge, w // merge
        br = torch.arange(mh, device=device)[:, None, None, None] * merge + torch.arange(merge, device=device)[None, None, :, None]
        bc = torch.arange(mw, device=device)[None, :, None, None] * merge + torch.arange(merge, device=device)[None, None, None, :]
        r = br.expand(mh, mw, merge, merge).reshape(-1).repeat(t)
        c = bc.expand(mh, mw, merge, merge).reshape(-1).repeat(t)
        rows.append(r)
        cols.append(c)
        img.append(torch.full_like(r, i))
    return torch.cat(rows), torch.cat(cols), torch.cat(img)


def vision_cu_seqlens(grid_thw, device=None) -> torch.Tensor:
    """Frame boundaries: each of the t frames of an image is one attention segment of h*w tokens."""
    lens = []
    for t, h, w in grid_thw:
        lens += [h * w] * t
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32, device=device)
    cu[1:] = torch.tensor(lens, dtype=torch.int32, device=device).cumsum(0)
    return cu


def _grid_list(grid_thw):
    if torch.is_tensor(grid_thw):
        return [tuple(int(x) for x in row) for row in grid_thw.tolist()]
    return [tuple(int(x) for x in row) for row in grid_thw]


class VisionMLP(nn.Module):
    def __init__(self, dim: int, hidden: int, act: str, **kw):
        super().__init__()
        self.linear_fc1 = Linear(dim, hidden, bias=True, **kw)
        self.linear_fc2 = Linear(hidden, dim, bias=True, **kw)
        self.act = act

    @scoped("vision_mlp")
    def forward(self, x):
        h = self.linear_fc1(x)
        h = Fn.gelu_tanh(h) if self.act in ("gelu_pytorch_tanh", "gelu_tanh") else F.gelu(h)
        return self.linear_fc2(h)


class VisionAttention(nn.Module):
    def __init__(self, dim: int, heads: int, **kw):
        super().__init__()
        self.H, self.Kd = heads, dim // heads
        self.qkv = Linear(dim, 3 * dim, bias=True, **kw)
        self.proj = Linear(dim, dim, bias=True, **kw)
        self.scale = self.Kd ** -0.5

    @scoped("vision_attention")
    def forward(self, x, cos, sin, cu_seqlens, max_seqlen: int):
        N = x.shape[0]
        qkv = self.qkv(x).view(N, 3, self.H, self.Kd)
        q = apply_vision_rope(qkv[:, 0], cos, sin).contiguous()
        k = apply_vision_rope(qkv[:, 1], cos, sin).contiguous()
        v = qkv[:, 2].contiguous()
        o = Fn.flash_attention(q, k, v, cu_seqlens, max_seqlen, scale=self.scale, causal=False)
        return self.proj(o.reshape(N, self.H * self.Kd))


class VisionBlock(nn.Module):
    def __init__(self, dim: int, hidden: int, heads: int, act: str, **kw):
        super().__init__()
        self.norm1 = LayerNorm(dim, 1e-6, **kw)
        self.norm2 = LayerNorm(dim, 1e-6, **kw)
        self.attn = VisionAttention(dim, heads, **kw)
        self.mlp = VisionMLP(dim, hidden, act, **kw)

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen):
        x = x + self.attn(self.norm1(x), cos, sin, cu_seqlens, max_seqlen)
        return x + self.mlp(self.norm2(x))


class VisionPatchMerger(nn.Module):
    """LayerNorm -> group 2x2 neighbours -> fc1 -> GELU -> fc2.  With ``postshuffle`` the norm
    runs over the grouped 4*dim vector instead of per patch."""

    def __init__(self, dim: int, merge: int, out_dim: int, postshuffle: bool = False, **kw):
        super().__init__()
        self.group = dim * merge * merge
        self.postshuffle = postshuffle
        self.norm = LayerNorm(self.group if postshuffle else dim, 1e-6, **kw)
        self.linear_fc1 = Linear(self.group, self.group, bias=True, **kw)
        self.linear_fc2 = Linear(self.group, out_dim, bias=True, **kw)

    @scoped("vision_merger")
    def forward(self, x):
        x = self.norm(x.reshape(-1, self.group) if self.postshuffle else x).reshape(-1, self.group)
        return self.linear_fc2(F.gelu(self.linear_fc1(x)))


class VisionTower(nn.Module):
    def __init__(self, *, depth, hidden_size, intermediate_size, num_heads, patch_size, temporal_patch_size,
                 spatial_merge_size, in_channels, out_hidden_size, num_position_embeddings,
                 hidden_act: str = "gelu_pytorch_tanh", deepstack_visual_indexes=(), device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.merge = spatial_merge_size
        self.hidden = hidden_size
        self.heads = num_heads
        self.in_features = in_channels * temporal_patch_size * patch_size * patch_size
        self.patch_embed = Linear(self.in_features, hidden_size, bias=True, **kw)
        self.pos_embed = nn.Parameter(torch.empty(num_position_embeddings, hidden_size, **kw))
        self.grid_side = int(math.isqrt(num_position_embeddings))
        self.blocks = nn.ModuleList(VisionBlock(hidden_size, intermediate_size, num_heads, hidden_act, **kw)
                                    for _ in range(depth))
        self.merger = VisionPatchMerger(hidden_size, spatial_merge_size, out_hidden_size, False, **kw)
        self.deepstack_visual_indexes = tuple(deepstack_visual_indexes)
        self.deepstack_mergers = nn.ModuleList(
            VisionPatchMerger(hidden_size, spatial_merge_size, out_hidden_size, True, **kw)
            for _ in self.deepstack_visual_indexes)
        self.reset_parameters()

    def reset_parameters(self):
        if self.pos_embed.device.type != "meta":
            nn.init.normal_(self.pos_embed, std=0.02)

    def interpolated_pos_embed(self, grid, device):
        """Bilinear interpolation of the learned sqrt(npos) x sqrt(npos) table to every image's
        (h, w) grid, repeated over frames and re-ordered into merge-block order."""
        side, m = self.grid_side, self.merge
        table = self.pos_embed
        outs = []
        for t, h, w in grid:
            hi = torch.linspace(0, side - 1, h, device=device)
            wi = torch.linspace(0, side - 1, w, device=device)
            h0, w0 = hi.floor().long(), wi.floor().long()
            h1, w1 = (h0 + 1).clamp(max=side - 1), (w0 + 1).clamp(max=side - 1)
            dh, dw = (hi - h0).to(table.dtype), (wi - w0).to(table.dtype)
            def flat(hh, ww):
                return (hh[:, None] * side + ww[None, :]).reshape(-1)
            idx4 = torch.stack([flat(h0, w0), flat(h0, w1), flat(h1, w0), flat(h1, w1)], dim=1)
            w4 = torch.stack([((1 - dh)[:, None] * (1 - dw)[None, :]).reshape(-1),
                              ((1 - dh)[:, None] * dw[None, :]).reshape(-1),
                              (dh[:, None] * (1 - dw)[None, :]).reshape(-1),
                              (dh[:, None] * dw[None, :]).reshape(-1)], dim=1)
            pe = Fn.gather4(table, idx4, w4)
            pe = pe.repeat(t, 1).view(t, h // m, m, w // m, m, -1).permute(0, 1, 3, 2, 4, 5).reshape(t * h * w, -1)
            outs.append(pe)
        return torch.cat(outs)

    def rotary(self, grid, device):
        """cos/sin [N, head_dim]: the first quarter of frequencies follows the row index, the
        second the column index, duplicated to fill the head (rotate-half layout)."""
        Kd = self.hidden // self.heads
        dim = Kd // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
        r, c, _ = token_spatial_coords(grid, self.merge, device)
        rot = torch.cat([r.float()[:, None] * inv, c.float()[:, None] * inv], dim=-1)  # [N, Kd/2]
        emb = torch.cat([rot, rot], dim=-1)
        return emb.cos(), emb.sin()

    @scoped("vision_model")
    def forward(self, pixel_values, grid_thw, cu_seqlens=None):
        grid = _grid_list(grid_thw)
        dev = pixel_values.device
        x = self.patch_embed(pixel_values.to(self.pos_embed.dtype))
        x = x + self.interpolated_pos_embed(grid, dev).to(x.dtype)
        cos, sin = self.rotary(grid, dev)
        if cu_seqlens is None:
            cu_seqlens = vision_cu_seqlens(grid, dev)
        max_len = max(h * w for _, h, w in grid)
        deep = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, cu_seqlens, max_len)
            if i in self.deepstack_visual_indexes:
                deep.append(self.deepstack_mergers[self.deepstack_visual_indexes.index(i)](x))
        merged = self.merger(x)
        if self.deepstack_visual_indexes:
            return merged, deep
        return merged
