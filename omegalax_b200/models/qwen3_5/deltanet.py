"""GatedDeltaNet linear-attention block (reference: omegalax/models/qwen3_5/deltanet.py).

    mixed = in_proj_qkv(x); z = in_proj_z(x); b = in_proj_b(x); a = in_proj_a(x)
    mixed = silu(causal_depthwise_conv1d(mixed, k=4))
    q, k, v = split(mixed);  beta = sigmoid(b);  g = -exp(A_log) * softplus(a + dt_bias)   (fp32)
    q, k heads repeated to the number of value heads; chunked gated delta rule in fp32
    out = out_proj(RMSNormGated(core, z))

Padded tokens are zeroed before the projections.  Tensor-parallel note: the fused
``in_proj_qkv`` output is ordered [all q | all k | all v]; a head-sharded layout therefore
has to permute the columns per rank so that every rank holds whole (q, k, v) head groups --
``tp_column_permutation`` returns that permutation.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import functional as Fn
from ...ops import reference as R
from ...parallel import tp as tp_lib
from ..qwen3.model import Linear
from .norms import RMSNormGated


from ...utils.profiling import scoped


def _l2norm(x, eps: float = 1e-6):
    return R.l2norm(x, eps)


def _causal_depthwise_conv1d(x_BCT, w_CK):
    return R.causal_conv1d(x_BCT, w_CK, activation_silu=False)


chunk_gated_delta_rule = R.chunk_gated_delta_rule


def tp_column_permutation(num_k_heads: int, num_v_heads: int, head_k: int, head_v: int, tp: int) -> torch.Tensor:
    """Column order of in_proj_qkv such that a contiguous 1/tp slice holds, for that rank's
    key heads, [q | k | v of the matching value heads]."""
    key_dim, rep = num_k_heads * head_k, num_v_heads // num_k_heads
    q_cols = torch.arange(key_dim).view(num_k_heads, head_k)
    k_cols = q_cols + key_dim
    v_cols = (torch.arange(num_v_heads * head_v) + 2 * key_dim).view(num_k_heads, rep * head_v)
    per = num_k_heads // tp
    out = []
    for r in range(tp):
        sl = slice(r * per, (r + 1) * per)
        out += [q_cols[sl].reshape(-1), k_cols[sl].reshape(-1), v_cols[sl].reshape(-1)]
    return torch.cat(out)


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg, device=None, dtype=None, tp_size: int = 1):
        """``tp_size`` > 1: this rank holds nk/tp key heads and the nv/tp value heads that read
        them (projection rows, conv channels, per-head decay parameters) and the matching input
        columns of the output projection; the head-dim norm weight is replicated."""
        super().__init__()
        D = cfg.hidden_size
        if cfg.linear_num_key_heads % tp_size or cfg.linear_num_value_heads % tp_size:
            raise ValueError(f"linear-attention heads ({cfg.linear_num_key_heads} k / {cfg.linear_num_value_heads} v) "
                             f"do not divide over tp_size={tp_size}")
        self.tp_size = tp_size
        self.nk, self.nv = cfg.linear_num_key_heads // tp_size, cfg.linear_num_value_heads // tp_size
        self.ak, self.av = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.key_dim, self.value_dim = self.nk * self.ak, self.nv * self.av
        self.conv_dim = 2 * self.key_dim + self.value_dim
        self.conv_k = cfg.linear_conv_kernel_dim
        kw = dict(device=device, dtype=dtype)
        self.in_proj_qkv = Linear(D, self.conv_dim, **kw)
        self.in_proj_z = Linear(D, self.value_dim, **kw)
        self.in_proj_b = Linear(D, self.nv, **kw)
        self.in_proj_a = Linear(D, self.nv, **kw)
        self.conv_weight = nn.Parameter(torch.empty(self.conv_dim, self.conv_k, **kw))
        self.dt_bias = nn.Parameter(torch.ones(self.nv, **kw))
        self.A_log = nn.Parameter(torch.empty(self.nv, **kw))
        self.norm = RMSNormGated(self.av, cfg.rms_norm_eps, **kw)
        self.out_proj = Linear(self.value_dim, D, **kw)
        if tp_size > 1:   # everything but the norm differs between tensor-parallel ranks
            self.tp_sharded = True
            for m in (self.in_proj_qkv, self.in_proj_z, self.in_proj_b, self.in_proj_a, self.out_proj):
                m.tp_sharded = True
        self.reset_parameters()

    def reset_parameters(self):
        if self.conv_weight.device.type == "meta":
            return
        with torch.no_grad():
            nn.init.normal_(self.conv_weight, std=1.0 / math.sqrt(self.conv_k))
            self.dt_bias.fill_(1.0)
            self.A_log.copy_(torch.log(torch.empty(self.nv).uniform_(0, 16).clamp_min(1e-4)))

    @scoped("gated_delta_net")
    def forward(self, x, ctx, residual=None):
        """x [M, D] packed rows of a [B, T] batch; ctx.segment_ids marks real tokens."""
        B, T = ctx.B, ctx.T
        tp = tp_lib.current() if self.tp_size > 1 else None
        if tp is not None:
            x = tp_lib.all_gather_rows(x, tp)      # sequence-parallel rows -> whole sequences, this rank's heads
        mask = (ctx.segment_ids != 0).reshape(-1, 1).to(x.dtype)
        x = x * mask
        mixed = self.in_proj_qkv(x).view(B, T, self.conv_dim)
        z = self.in_proj_z(x)
        b = self.in_proj_b(x)
        a = self.in_proj_a(x)
        mixed = Fn.causal_conv1d_silu(mixed, self.conv_weight)
        q, k, v = torch.split(mixed, [self.key_dim, self.key_dim, self.value_dim], dim=-1)
        q = q.reshape(B, T, self.nk, self.ak)
        k = k.reshape(B, T, self.nk, self.ak)
        v = v.reshape(B, T, self.nv, self.av)
        beta = torch.sigmoid(b.float()).view(B, T, self.nv)
        g = (-torch.exp(self.A_log.float()) * F.softplus(a.float() + self.dt_bias.float())).view(B, T, self.nv)
        core = Fn.gated_delta_rule(q, k, v, g, beta)               # key heads are shared by nv/nk value heads

        core = self.norm(core.reshape(-1, self.av), z.reshape(-1, self.av))
        if tp is not None:
            return tp_lib.row_parallel_linear(core.reshape(B * T, self.value_dim), self.out_proj.weight, residual, tp)
        return self.out_proj(core.reshape(B * T, self.value_dim), residual=residual)
