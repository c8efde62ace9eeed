"""Plain-PyTorch definitions of every op (fp32 arithmetic where the model contract asks
for it).  They run on CPU and GPU, are the oracle of the kernel tests, and are the path
taken for non-bf16 or non-CUDA tensors.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x, w, eps: float, one_plus: bool = False, scale_in_dtype: bool = False):
    """RMSNorm.  ``one_plus`` multiplies by ``1 + w`` (Qwen3.5).  ``scale_in_dtype``
    casts the normalised value to the input dtype before the scale (Qwen3-VL text)."""
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if scale_in_dtype:
        return n.to(x.dtype) * (w.to(x.dtype) if not one_plus else (1.0 + w).to(x.dtype))
    wf = w.float()
    if one_plus:
        wf = 1.0 + wf
    return (n * wf).to(x.dtype)


def rmsnorm_gated(x, w, z, eps: float):
    """weight * norm(x) (cast to x.dtype) * silu(z in fp32)."""
    xf = x.float()
    n = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
    n = w.to(x.dtype) * n
    return (n.float() * F.silu(z.float())).to(x.dtype)


def layernorm(x, w, b, eps: float):
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), eps).to(x.dtype)


def swiglu(gu):
    g, u = gu.chunk(2, dim=-1)
    return F.silu(g.float()).mul(u.float()).to(gu.dtype) if gu.dtype != torch.float32 else F.silu(g) * u


def rope_tables(positions, head_dim: int, theta: float):
    """fp32 sin/cos of shape positions.shape + (head_dim/2,)."""
    inv = theta ** (-(torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device) / head_dim))
    ang = positions.to(torch.float32)[..., None] * inv
    return torch.sin(ang), torch.cos(ang)


def apply_rope(x, sin, cos, rot: int | None = None):
    """Half-split rotation of the first ``rot`` channels of x [..., heads, K]; sin/cos are
    [..., rot/2] and broadcast over heads.  Arithmetic in x.dtype (tables are cast)."""
    K = x.shape[-1]
    rot = K if rot is None else rot
    s = sin.to(x.dtype).unsqueeze(-2)
    c = cos.to(x.dtype).unsqueeze(-2)
    xr = x[..., :rot]
    x1, x2 = xr[..., : rot // 2], xr[..., rot // 2:]
    out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    if rot < K:
        out = torch.cat([out, x[..., rot:]], dim=-1)
    return out


def attention(q, k, v, *, causal: bool, scale: float, k_start=None, k_end=None, kv_mask=None):
    """Exact softmax attention with GQA.  q [B,T,H,K], k/v [B,S,G,K].

    ``k_start``/``k_end`` ([B,T] int): query t only sees keys in [k_start, k_end).
    ``kv_mask`` [B,S] bool: keys that exist.  fp32 softmax; output in q.dtype.
    With ``causal`` and T != S, query t sits at key position t + (S - T).
    """
    B, T, H, K = q.shape
    S, G = k.shape[1], k.shape[2]
    R = H // G
    qf = q.float().view(B, T, G, R, K)
    kf, vf = k.float(), v.float()
    logits = torch.einsum("btgrk,bsgk->bgrts", qf, kf) * scale
    mask = torch.ones(B, T, S, dtype=torch.bool, device=q.device)
    kpos = torch.arange(S, device=q.device)
    if causal:
        qpos = torch.arange(T, device=q.device) + (S - T)
        mask &= (kpos[None, :] <= qpos[:, None])[None]
    if k_start is not None:
        mask &= kpos[None, None, :] >= k_start[:, :, None]
    if k_end is not None:
        mask &= kpos[None, None, :] < k_end[:, :, None]
    if kv_mask is not None:
        mask &= kv_mask[:, None, :]
    logits = logits.masked_fill(~mask[:, None, None], torch.finfo(torch.float32).min)
    p = torch.softmax(logits, dim=-1)
    p = p * mask[:, None, None].any(-1, keepdim=True)  # fully masked rows give zeros
    out = torch.einsum("bgrts,bsgk->btgrk", p, vf).reshape(B, T, H, K)
    return out.to(q.dtype)


def attention_varlen(q, k, v, cu_seqlens, *, causal: bool, scale: float):
    """Packed rows: q [N,H,K], k/v [N,G,K]; block-diagonal over the sequences."""
    outs = []
    cu = cu_seqlens.tolist()
    for a, b in zip(cu[:-1], cu[1:]):
        if b > a:
            outs.append(attention(q[None, a:b], k[None, a:b], v[None, a:b], causal=causal, scale=scale)[0])
    return torch.cat(outs, dim=0) if outs else q.new_zeros(q.shape)


def cross_entropy_sum(hidden, w_lm, targets, mask):
    """sum over rows of mask * nll(logits = hidden @ w_lm^T), fp32 log-sum-exp."""
    logits = (hidden @ w_lm.to(hidden.dtype).t()).float()
    lse = torch.logsumexp(logits, dim=-1)
    tl = logits.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1)
    return ((lse - tl) * mask.float()).sum()


def l2norm(x, eps: float = 1e-6):
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def causal_conv1d(x_bct, w_ck, activation_silu: bool = True):
    """Depthwise causal conv over time.  x [B,C,T], w [C,K]: left pad K-1."""
    K = w_ck.shape[-1]
    y = F.conv1d(F.pad(x_bct, (K - 1, 0)), w_ck.unsqueeze(1).to(x_bct.dtype), groups=x_bct.shape[1])
    return F.silu(y) if activation_silu else y


def chunk_gated_delta_rule(q, k, v, g, beta, chunk: int = 64, initial_state=None, output_final_state=False):
    """Chunked gated delta rule in fp32.  q,k [B,T,H,A]; v [B,T,H,U]; g,beta [B,T,H].

    Per head: S_t = S_{t-1} exp(g_t) + k_t (beta_t (v_t - S_{t-1}^T exp(g_t) k_t))^T and
    o_t = S_t^T q_t, evaluated chunk by chunk with an in-chunk triangular solve.
    q and k are L2-normalised and q is scaled by A**-0.5 first.
    """
    dt = q.dtype
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    q = l2norm(q)
    k = l2norm(k)
    B, T, H, A = q.shape
    U = v.shape[-1]
    q = q * (A ** -0.5)
    pad = (-T) % chunk
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
        g, beta = (F.pad(t, (0, 0, 0, pad)) for t in (g, beta))
    Tp = T + pad
    J = Tp // chunk
    # [B,H,J,C,*]
    q, k, v = (t.permute(0, 2, 1, 3).reshape(B, H, J, chunk, -1) for t in (q, k, v))
    g, beta = (t.permute(0, 2, 1).reshape(B, H, J, chunk) for t in (g, beta))
    g = g.cumsum(-1)
    decay = torch.tril(torch.exp(torch.tril(g[..., :, None] - g[..., None, :])))
    kb = k * beta[..., None]
    vb = v * beta[..., None]
    strict = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), -1)
    attn = -(kb @ k.transpose(-1, -2)) * decay
    attn = attn.masked_fill(~strict, 0.0)
    eye = torch.eye(chunk, device=q.device, dtype=torch.float32)
    # (I - attn)^-1 via a unit-lower-triangular solve
    Tm = torch.linalg.solve_triangular(eye - attn, eye.expand_as(attn).contiguous(), upper=False, unitriangular=True)
    v_corr = Tm @ vb
    k_cum = Tm @ (kb * torch.exp(g)[..., None])
    S = q.new_zeros(B, H, A, U) if initial_state is None else initial_state.float().clone()
    outs = []
    incl = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device))
    for j in range(J):
        qj, kj, gj = q[:, :, j], k[:, :, j], g[:, :, j]
        intra = (qj @ kj.transpose(-1, -2)) * decay[:, :, j]
        intra = intra.masked_fill(~incl, 0.0)
        v_new = v_corr[:, :, j] - k_cum[:, :, j] @ S
        o = (qj * torch.exp(gj)[..., None]) @ S + intra @ v_new
        outs.append(o)
        gl = gj[..., -1]
        S = S * torch.exp(gl)[..., None, None] + (kj * torch.exp(gl[..., None] - gj)[..., None]).transpose(-1, -2) @ v_new
    o = torch.stack(outs, dim=2).reshape(B, H, Tp, U)[:, :, :T].permute(0, 2, 1, 3)
    o = o.to(dt)
    if output_final_state:
        return o, S
    return o


def recurrent_gated_delta_rule(q, k, v, g, beta, initial_state=None):
    """Token-by-token form of the same recurrence (decode path and test oracle)."""
    dt = q.dtype
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    q = l2norm(q)
    k = l2norm(k)
    B, T, H, A = q.shape
    U = v.shape[-1]
    q = q * (A ** -0.5)
    S = q.new_zeros(B, H, A, U) if initial_state is None else initial_state.float().clone()
    outs = []
    for t in range(T):
        S = S * torch.exp(g[:, t])[..., None, None]
        kv = torch.einsum("bha,bhau->bhu", k[:, t], S)
        delta = (v[:, t] - kv) * beta[:, t][..., None]
        S = S + torch.einsum("bha,bhu->bhau", k[:, t], delta)
        outs.append(torch.einsum("bha,bhau->bhu", q[:, t], S))
    return torch.stack(outs, dim=1).to(dt), S


def gelu_tanh(x):
    return F.gelu(x, approximate="tanh")
