"""Qwen3-VL: ViT with DeepStack taps + Qwen3-style decoder with interleaved 3-D MRoPE
(reference: omegalax/models/qwen3_vl/model.py)."""
from __future__ import annotations

import dataclasses

import numpy as np
import torch
from torch import nn

from ...ops import functional as Fn
from ...ops import reference as R
from ...parallel import tp as tp_lib
from ..qwen3.model import DecoderLayer, Embedding, ForwardCtx, Linear, left_pad_cu_seqlens, vocab_parallel_head
from ..qwen3.norms import RMSNorm
from ..qwen3_5.rope import interleave_mrope
from .config import Qwen3VLConfig
from .vision import VisionModel


def apply_rope(x, sin, cos):
    return R.apply_rope(x, sin, cos)


def compute_mrope_pos_embeddings(position_ids_ZBT, head_dim: int, theta: float, mrope_section):
    """fp32 (sin, cos), each [B, T, head_dim/2]: full-head rotation; frequency slot i follows
    the height position if i in {1,4,7,..} and i < 3*sec[1], the width position if i in
    {2,5,8,..} and i < 3*sec[2], else the temporal position."""
    inv = theta ** (-(torch.arange(0, head_dim, 2, dtype=torch.float32, device=position_ids_ZBT.device) / head_dim))
    freqs = position_ids_ZBT.to(torch.float32)[..., None] * inv
    f = interleave_mrope(freqs, mrope_section)
    return torch.sin(f), torch.cos(f)


def get_rope_index(input_ids, image_grid_thw=None, video_grid_thw=None, attention_mask=None,
                   spatial_merge_size: int = 2, image_token_id: int = 0, video_token_id: int = 0,
                   vision_start_token_id: int = 0):
    """3-D position ids for MRoPE on the host (numpy).  Text tokens advance all three axes
    together; a vision span of grid (t, h, w) uses its (t, h/m, w/m) grid indices offset by the
    running maximum + 1.  Videos are split into per-frame grids.  Returns (position_ids
    [3,B,T] int64, rope_deltas [B,1])."""
    ids = np.asarray(input_ids)
    mask = np.ones_like(ids) if attention_mask is None else np.asarray(attention_mask)
    images = [] if image_grid_thw is None else [tuple(int(v) for v in row) for row in np.asarray(image_grid_thw).tolist()]
    videos = []
    if video_grid_thw is not None:
        for t, h, w in np.asarray(video_grid_thw).tolist():
            videos += [(1, int(h), int(w))] * int(t)
    B, T = ids.shape
    out = np.zeros((3, B, T), dtype=np.int64)
    deltas = []
    ii = vi = 0
    m = spatial_merge_size
    for b in range(B):
        row = ids[b][mask[b] == 1]
        n = row.shape[0]
        pos = np.zeros((3, n), dtype=np.int64)
        starts = np.where(row == vision_start_token_id)[0]
        starts = starts[starts + 1 < n]
        kinds = row[starts + 1]
        n_img, n_vid = int((kinds == image_token_id).sum()), int((kinds == video_token_id).sum())
        cursor = 0      # next token to place
        nxt = 0         # next free position value
        for _ in range(n_img + n_vid):
            rest = row[cursor:]
            e_img = int(np.argmax(rest == image_token_id)) + cursor if (n_img > 0 and (rest == image_token_id).any()) else n + 1
            e_vid = int(np.argmax(rest == video_token_id)) + cursor if (n_vid > 0 and (rest == video_token_id).any()) else n + 1
            if e_img < e_vid:
                t, h, w = images[ii]; ii += 1; n_img -= 1; e = e_img
            else:
                t, h, w = videos[vi]; vi += 1; n_vid -= 1; e = e_vid
            gh, gw = h // m, w // m
            tl = e - cursor
            pos[:, cursor:e] = nxt + np.arange(tl)[None, :]
            base = nxt + tl
            span = t * gh * gw
            tt = np.repeat(np.arange(t), gh * gw)
            hh = np.tile(np.repeat(np.arange(gh), gw), t)
            ww = np.tile(np.arange(gw), t * gh)
            pos[:, e:e + span] = np.stack([tt, hh, ww]) + base
            cursor = e + span
            nxt = int(pos[:, :cursor].max()) + 1 if cursor > 0 else 0
        if cursor < n:
            pos[:, cursor:] = nxt + np.arange(n - cursor)[None, :]
        out[:, b, mask[b] == 1] = pos
        deltas.append(int(pos.max()) + 1 - T if n > 0 else 0)
    return out, np.asarray(deltas, dtype=np.int64).reshape(-1, 1)


class TextMLP(nn.Module):
    """Alias kept for API parity; the decoder layers use the shared SwiGLU module."""


@dataclasses.dataclass(frozen=True)
class _TextCfgShim:
    """View of a Qwen3VLConfig with the attribute names the shared decoder layer reads.  The
    auxiliary router loss of this family carries no coefficient (omegalax/models/qwen3_vl/model.py:282)."""
    base: Qwen3VLConfig

    def __getattr__(self, name):
        if name == "aux_loss_coef":
            return 1.0
        return getattr(object.__getattribute__(self, "base"), name)

    def is_moe_layer(self, i):
        return self.base.is_moe_layer(i)


class Qwen3VL(nn.Module):
    def __init__(self, cfg: Qwen3VLConfig, device=None, dtype=None, tp_size: int = 1):
        """``tp_size`` > 1 splits the text decoder (heads, MLP width) over tensor-parallel ranks
        with sequence-parallel activations between the blocks; the vision tower, the embedding
        and the head are replicated (each rank back-propagates only its rows into them and the
        engine sums those gradients over the tensor-parallel group)."""
        super().__init__()
        self.cfg = cfg
        self.tp_size = tp_size
        dtype = dtype or torch.float32
        kw = dict(device=device, dtype=dtype)
        shim = _TextCfgShim(cfg)
        self.visual = VisionModel(cfg.vision, **kw)
        self.embedder = Embedding(cfg.vocab_size, cfg.emb_dim, **kw)
        self.layers = nn.ModuleList(DecoderLayer(shim, i, tp_size=tp_size, **kw) for i in range(cfg.num_layers))
        self.final_norm = RMSNorm(cfg.emb_dim, cfg.norm_eps, **kw)
        self.vocab_parallel = vocab_parallel_head(cfg, tp_size)   # untied head: split over the vocabulary
        self.lm_head = Linear(cfg.emb_dim, cfg.vocab_size // tp_size if self.vocab_parallel else cfg.vocab_size, **kw)
        self.lm_head.tp_sharded = self.vocab_parallel
        self.layer_runner = None
        self._attn_backend = "sm100"

    def train_units(self):
        return [("visual", [self.visual]), ("embedder", [self.embedder])] + \
               [(f"layers.{i}", [l]) for i, l in enumerate(self.layers)] + [("head", [self.final_norm, self.lm_head])]

    def forward(self, token_ids, attention_mask=None, position_ids_ZBT=None, pixel_values=None,
                image_grid_thw=None, vision_cu_seqlens=None, return_local_rows: bool = False):
        """Hidden states [B,T,D] before the head and the summed router loss.  Under tensor
        parallelism ``return_local_rows`` returns this rank's rows [B*T/tp, D] of the flattened
        token rows instead of gathering them (the trainer scores them in place)."""
        B, T = token_ids.shape
        dev = token_ids.device
        if attention_mask is None:
            attention_mask = torch.ones_like(token_ids)
        x = self.embedder(token_ids.reshape(-1))
        deep, vis_pos, vis_ok = [], None, None
        if pixel_values is not None and pixel_values.numel() > 0:
            if vision_cu_seqlens is None:
                raise ValueError("vision_cu_seqlens is required when pixel_values are given")
            feats, deep = self.visual(pixel_values.to(x.dtype), image_grid_thw, vision_cu_seqlens.to(torch.int32))
            is_img = token_ids.reshape(-1) == self.cfg.image_token_id
            if is_img.is_cuda:
                # no host synchronisation: the first n image-token positions by a stable sort; when the
                # (padded) feature rows outnumber the image tokens the surplus rows are made no-ops
                vis_pos, vis_ok = Fn.first_true_rows(is_img, feats.shape[0])
                src = torch.where(vis_ok, feats[: vis_pos.numel()].to(x.dtype), x.index_select(0, vis_pos))
                x = Fn.scatter_rows(x, vis_pos, src, replace=True)
            else:
                vis_ok = None
                vis_pos = torch.nonzero(is_img, as_tuple=False).squeeze(-1)[: feats.shape[0]]
                x = Fn.scatter_rows(x, vis_pos, feats[: vis_pos.numel()].to(x.dtype), replace=True)
        if position_ids_ZBT is None:
            pos = (attention_mask.cumsum(-1) - 1).clamp_min(0) * (attention_mask != 0)
            position_ids_ZBT = pos[None].expand(3, B, T)
        sin, cos = compute_mrope_pos_embeddings(position_ids_ZBT, self.cfg.head_dim, self.cfg.rope_theta,
                                                self.cfg.mrope_section)
        seg = (attention_mask != 0).to(torch.int32)
        first = (seg.cumsum(-1) == 0).sum(-1)
        ctx = ForwardCtx(B=B, T=T, sin=sin.reshape(B * T, -1), cos=cos.reshape(B * T, -1),
                         cu_seqlens=left_pad_cu_seqlens(first, B, T), segment_ids=seg,
                         k_start=first.to(torch.int64), positions=position_ids_ZBT)
        tp = tp_lib.current() if self.tp_size > 1 else None
        if tp is not None:
            if (B * T) % tp.size:
                raise ValueError("tensor parallelism needs B*T divisible by tp_size")
            m = B * T // tp.size
            x = x[tp.rank * m:(tp.rank + 1) * m]              # sequence-parallel rows of this rank
            if vis_pos is not None:
                # image rows that fall outside this rank's slice add zeros to its first row
                mine = (vis_pos >= tp.rank * m) & (vis_pos < (tp.rank + 1) * m)
                vis_ok = mine.unsqueeze(-1) if vis_ok is None else (vis_ok & mine.unsqueeze(-1))
                vis_pos = torch.where(mine, vis_pos - tp.rank * m, torch.zeros_like(vis_pos))
        aux_total = torch.zeros((), dtype=torch.float32, device=x.device)
        for i, layer in enumerate(self.layers):
            if self.layer_runner is not None:
                x, aux = self.layer_runner(layer, x, ctx)
            else:
                x, aux = layer(x, ctx)
            aux_total = aux_total + aux
            if vis_pos is not None and i < len(deep):  # DeepStack: add tapped vision features
                d = deep[i][: vis_pos.numel()].to(x.dtype)
                d = d if vis_ok is None else d * vis_ok.to(x.dtype)
                # under tp the masked-out rows all point at row 0: index_add tolerates the repeats,
                # the row-scatter kernel wants unique rows
                x = x.index_add(0, vis_pos, d) if tp is not None else Fn.scatter_rows(x, vis_pos, d)
        x = self.final_norm(x)
        if tp is not None:
            if return_local_rows:
                return x, aux_total
            x = tp_lib.all_gather_rows(x, tp)
        return x.view(B, T, -1), aux_total
