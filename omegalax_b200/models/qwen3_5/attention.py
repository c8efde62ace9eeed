"""Gated full attention of Qwen3.5 (reference: omegalax/models/qwen3_5/attention.py).

The query projection emits, per head, [q | gate]; q and k get a (1+w) RMSNorm over the head
dimension and partial interleaved MRoPE; causal attention; the output is multiplied by
sigmoid(gate) before the output projection.
"""
from __future__ import annotations

import torch
from torch import nn

from ...ops import functional as Fn
from ...ops import reference as R
from ...parallel import tp as tp_lib
from ..qwen3.model import Linear
from .norms import RMSNorm


from ...utils.profiling import scoped


class Attention(nn.Module):
    def __init__(self, cfg, device=None, dtype=None, tp_size: int = 1):
        super().__init__()
        if cfg.num_attention_heads % tp_size or cfg.num_key_value_heads % tp_size:
            raise ValueError(f"heads ({cfg.num_attention_heads} q / {cfg.num_key_value_heads} kv) do not divide "
                             f"over tp_size={tp_size}")
        if tp_size > 1 and cfg.attention_bias:
            raise ValueError("tensor-parallel attention with projection biases is not supported")
        H, G = cfg.num_attention_heads // tp_size, cfg.num_key_value_heads // tp_size
        Kd, D = cfg.head_dim, cfg.hidden_size
        self.tp_size = tp_size
        self.H, self.G, self.Kd = H, G, Kd
        self.rot = int(Kd * cfg.partial_rotary_factor)
        kw = dict(device=device, dtype=dtype)
        # fused rows: [per head (q | gate)] then k heads then v heads
        self.qkv_proj = Linear(D, (2 * H + 2 * G) * Kd, bias=cfg.attention_bias, **kw)
        self.o_proj = Linear(H * Kd, D, bias=cfg.attention_bias, **kw)
        self.q_norm = RMSNorm(Kd, cfg.rms_norm_eps, **kw)
        self.k_norm = RMSNorm(Kd, cfg.rms_norm_eps, **kw)
        self.eps = cfg.rms_norm_eps
        self.scale = Kd ** -0.5
        self.qkv_proj.tp_sharded = self.o_proj.tp_sharded = tp_size > 1

    @scoped("attention")
    def forward(self, x, ctx, residual=None):
        tp = tp_lib.current() if self.tp_size > 1 else None
        if tp is not None:
            x = tp_lib.all_gather_rows(x, tp)      # sequence-parallel rows -> all rows, this rank's heads
        M = x.shape[0]
        B, T = ctx.B, ctx.T
        qkv = self.qkv_proj(x)
        q, k, v, gate = Fn.qk_norm_rope(qkv, self.q_norm.weight, self.k_norm.weight, ctx.sin, ctx.cos,
                                        self.H, self.G, self.Kd, rot=self.rot, eps=self.eps, one_plus=True,
                                        q_stride_heads=2)
        if Fn.use_kernels(q) or (Fn.library_mode() and q.is_cuda):
            # own flash-attention kernels for 64-, 128- and 256-wide heads (the published configs use 256)
            o = Fn.flash_attention(q, k, v, ctx.cu_seqlens, T, scale=self.scale, causal=True)
        else:
            ks = None if ctx.k_start is None else ctx.k_start[:, None].expand(B, T)
            o = R.attention(q.reshape(B, T, self.H, self.Kd), k.reshape(B, T, self.G, self.Kd),
                            v.reshape(B, T, self.G, self.Kd), causal=True, scale=self.scale,
                            k_start=ks).reshape(M, self.H, self.Kd)
        o = Fn.sigmoid_gate(o, gate)
        if tp is not None:
            return tp_lib.row_parallel_linear(o.reshape(M, self.H * self.Kd), self.o_proj.weight, residual, tp)
        return self.o_proj(o.reshape(M, self.H * self.Kd), residual=residual)
