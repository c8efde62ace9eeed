"""Differentiable ops used by the models.

Each op has two implementations: the hand-written sm_100a kernels (taken for CUDA bf16
tensors) and the plain-PyTorch definition in ``reference.py`` (CPU, fp32, oracle).  On a
CUDA bf16 tensor the kernel path is the only one; there is no silent fallback.

Weight gradients: when a weight tensor carries a ``main_grad`` attribute (an fp32 buffer
owned by the sharded train state), the backward accumulates straight into it with the
GEMM's fp32-accumulate epilogue and returns no autograd gradient for the weight.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from . import kernels as K
from . import reference as R

bf16 = torch.bfloat16


class _Stash:
    """Selective rematerialisation: tagged op outputs recorded during the no-grad forward of a
    layer are replayed (instead of recomputed) when the layer is re-run for its backward."""

    def __init__(self, tags):
        # a tag written "name!" marks an op whose output value nothing in the layer's backward
        # needs (the layer's last projection): it is neither stored nor recomputed, the replay
        # gets an uninitialised tensor of the right shape
        self.skip = frozenset(t[:-1] for t in tags if t.endswith("!"))
        self.tags = frozenset(t.rstrip("!") for t in tags)
        self.items: dict = {}
        self.mode = "off"      # "record" | "replay" | "off"
        self.counter: dict = {}

    def key(self, tag):
        i = self.counter.get(tag, 0)
        self.counter[tag] = i + 1
        return (tag, i)


_ACTIVE_STASH: "_Stash | None" = None


class stash_scope:
    def __init__(self, stash, mode):
        self.stash, self.mode = stash, mode

    def __enter__(self):
        global _ACTIVE_STASH
        self.prev = _ACTIVE_STASH
        if self.stash is not None:
            self.stash.mode = self.mode
            self.stash.counter = {}
        _ACTIVE_STASH = self.stash
        return self.stash

    def __exit__(self, *a):
        global _ACTIVE_STASH
        if self.stash is not None:
            self.stash.mode = "off"
        _ACTIVE_STASH = self.prev


def _stash_lookup(tag):
    """(key, stored value or None) for a tagged call under the active stash."""
    st = _ACTIVE_STASH
    if st is None or tag is None or tag not in st.tags or st.mode == "off":
        return None, None
    k = st.key(tag)
    if tag in st.skip:
        return k, (_SKIP if st.mode == "replay" else None)
    return k, (st.items.get(k) if st.mode == "replay" else None)


_SKIP = object()


def _stash_store(key, value):
    st = _ACTIVE_STASH
    if st is not None and key is not None and st.mode == "record" and key[0] not in st.skip:
        st.items[key] = value


def library_mode() -> bool:
    """``OMEGALAX_B200_OPS=library``: the stand-in baseline.  No kernel of this repository runs;
    every op is the PyTorch library call a plain PyTorch program would make (cuBLAS through
    ``F.linear``, flash SDPA, eager elementwise ops, a row-chunked checkpointed cross-entropy) and
    the engine moves parameters and gradients with NCCL collectives."""
    return os.environ.get("OMEGALAX_B200_OPS") == "library"


def use_kernels(t: torch.Tensor) -> bool:
    return (t.is_cuda and t.dtype == bf16 and os.environ.get("OMEGALAX_B200_REFERENCE_OPS") != "1"
            and not library_mode())


def _sdpa_packed(q, k, v, cu_seqlens, max_seqlen: int, scale: float, causal: bool):
    """Library attention on packed rows: one flash SDPA call when every sequence has max_seqlen rows
    (the training batches), else one call per sequence."""
    N, H, Kd = q.shape
    G = k.shape[1]
    B = cu_seqlens.numel() - 1
    sdpa = torch.nn.functional.scaled_dot_product_attention
    if N == B * max_seqlen:
        o = sdpa(q.view(B, max_seqlen, H, Kd).transpose(1, 2), k.reshape(B, max_seqlen, G, Kd).transpose(1, 2),
                 v.reshape(B, max_seqlen, G, Kd).transpose(1, 2), is_causal=bool(causal), scale=scale, enable_gqa=True)
        return o.transpose(1, 2).reshape(N, H, Kd)
    outs = []
    cu = cu_seqlens.tolist()
    for a, b in zip(cu[:-1], cu[1:]):
        if b > a:
            o = sdpa(q[a:b].transpose(0, 1)[None], k[a:b].transpose(0, 1)[None], v[a:b].transpose(0, 1)[None],
                     is_causal=bool(causal), scale=scale, enable_gqa=True)
            outs.append(o[0].transpose(0, 1))
    return torch.cat(outs, dim=0) if outs else q.new_zeros(q.shape)


def _acc_main_grad(w, fn_into, fn_new):
    """Accumulate into w.main_grad when present (returns None), else return a new grad."""
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        fn_into(mg)
        return None
    return fn_new()


# ----------------------------------------------------------------------------- linear
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual, y_pre=None, bias=None):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        y = y_pre
        ag = getattr(w, "ag_spec", None)
        if y is None and ag is not None and bias is None:   # sharded weight gathered inside this GEMM's launch
            y = ag.run(x2.contiguous(), w, residual)
        if y is None:
            y = K.gemm(x2, w, residual=residual, bias=bias)   # bias and residual are added in the GEMM epilogue
        ctx.save_for_backward(x2, w)
        ctx.shp = shp
        ctx.has_res = residual is not None
        ctx.has_bias = bias is not None
        ctx.w_ref = w
        return y.view(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        w_obj = ctx.w_ref
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = K.gemm(dy2, w, b_mn=True).view(ctx.shp)
        dw = None
        pg = getattr(w_obj, "peer_grad", None)
        if ctx.needs_input_grad[1] and pg is not None:
            K.gemm_peer_reduce(dy2, x2, pg[0], pg[1], pg[2], a_mn=True, b_mn=True)
        elif ctx.needs_input_grad[1]:
            dw = _acc_main_grad(
                w_obj,
                lambda mg: K.gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=True),
                lambda: K.gemm(dy2, x2, a_mn=True, b_mn=True),
            )
        db = dy2.sum(0) if (ctx.has_bias and ctx.needs_input_grad[4]) else None
        return dx, dw, (dy if ctx.has_res else None), None, db


def linear(x, w, residual=None, bias=None, tag=None):
    """y = x @ w.T (+ bias) (+ residual); w is [out, in]."""
    if use_kernels(x) and w.dtype == bf16 and w.shape[0] % 8:
        # narrow heads (a 1-row gate, a handful of per-head scalars): the GEMM tiles need rows in
        # multiples of 8, so run on a zero-padded weight and drop the padding columns
        n = w.shape[0]
        y = linear(x, F.pad(w, (0, 0, 0, 8 - n % 8)), None, None if bias is None else F.pad(bias, (0, 8 - n % 8)))
        y = y[..., :n]
        return y if residual is None else y + residual
    if use_kernels(x) and w.dtype == bf16:
        key, pre = _stash_lookup(tag if bias is None else None)
        if pre is _SKIP:
            pre = torch.empty(x.numel() // x.shape[-1], w.shape[0], dtype=x.dtype, device=x.device)
        fused_bias = bias is not None and bias.dtype == bf16 and bias.is_contiguous()
        y = _LinearFn.apply(x, w, residual if (bias is None or fused_bias) else None,
                            None if pre is None else pre.view(-1, w.shape[0]), bias if fused_bias else None)
        _stash_store(key, y)
        if bias is not None and not fused_bias:
            y = y + bias
            if residual is not None:
                y = y + residual
        return y
    y = torch.nn.functional.linear(x, w.to(x.dtype), None if bias is None else bias.to(x.dtype))
    if residual is not None:
        y = y + residual
    return y


# ----------------------------------------------------------------------------- rmsnorm
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, one_plus):
        y, rstd = K.rmsnorm_fwd(x, w, eps, one_plus)
        ctx.save_for_backward(x, w, rstd)
        ctx.eps, ctx.one_plus, ctx.w_ref = eps, one_plus, w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        mg = getattr(ctx.w_ref, "main_grad", None)
        if mg is not None:
            dx = K.rmsnorm_bwd(dy, x, w, rstd, ctx.eps, mg, ctx.one_plus)
            return dx, None, None, None
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        dx = K.rmsnorm_bwd(dy, x, w, rstd, ctx.eps, dw, ctx.one_plus)
        return dx, dw.to(w.dtype), None, None


def rmsnorm(x, w, eps: float, one_plus: bool = False, scale_in_dtype: bool = False):
    if use_kernels(x) and w.dtype == bf16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        return _RMSNormFn.apply(x, w, eps, one_plus)
    return R.rmsnorm(x, w, eps, one_plus, scale_in_dtype)


class _GatedRMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, z, eps):
        y, rstd = K.gated_rmsnorm_fwd(x, z, w, eps)
        ctx.save_for_backward(x, w, z, rstd)
        ctx.eps, ctx.w_ref = eps, w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, z, rstd = ctx.saved_tensors
        mg = getattr(ctx.w_ref, "main_grad", None)
        dwf = mg if mg is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        dx, dz = K.gated_rmsnorm_bwd(dy.contiguous(), x, z, w, rstd, ctx.eps, dwf)
        return dx, (None if mg is not None else dwf.to(w.dtype)), dz, None


def rmsnorm_gated(x, w, z, eps: float):
    """weight * norm(x) in the input dtype, times silu(z) in fp32; x, z [M, D]."""
    if use_kernels(x) and w.dtype == bf16 and x.dim() == 2 and x.shape[-1] in (128, 256):
        return _GatedRMSNormFn.apply(x.contiguous(), w, z.contiguous(), eps)
    return R.rmsnorm_gated(x, w, z, eps)


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        y, mean, rstd = K.layernorm_fwd(x, w, b, eps)
        ctx.save_for_backward(x, w, mean, rstd)
        ctx.w_ref, ctx.b_ref = w, b
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, mean, rstd = ctx.saved_tensors
        mgw, mgb = getattr(ctx.w_ref, "main_grad", None), getattr(ctx.b_ref, "main_grad", None)
        fused = mgw is not None and mgb is not None
        dwf = mgw if fused else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        dbf = mgb if fused else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        dx = K.layernorm_bwd(dy.contiguous(), x, w, mean, rstd, dwf, dbf)
        if fused:
            return dx, None, None, None
        return dx, dwf.to(w.dtype), dbf.to(w.dtype), None


def layernorm(x, w, b, eps: float):
    """LayerNorm with bias over the last dim, fp32 statistics."""
    D = x.shape[-1]
    if use_kernels(x) and w.dtype == bf16 and b.dtype == bf16 and D % 8 == 0 and D <= 2048:
        return _LayerNormFn.apply(x.reshape(-1, D).contiguous(), w, b, eps).view(x.shape)
    return R.layernorm(x, w, b, eps)


# ----------------------------------------------------------------------------- gelu, row gather / scatter
class _GeluTanhFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return K.gelu_tanh_fwd(x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return K.gelu_tanh_bwd(x, dy.contiguous())


def gelu_tanh(x):
    if use_kernels(x) and x.numel() % 8 == 0:
        return _GeluTanhFn.apply(x.contiguous())
    return R.gelu_tanh(x)


class _ScatterRowsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos32, src, replace):
        out = x.clone()
        K.scatter_rows_(out, pos32, src, replace)
        ctx.save_for_backward(pos32)
        ctx.replace = replace
        return out

    @staticmethod
    def backward(ctx, dy):
        (pos32,) = ctx.saved_tensors
        dy = dy.contiguous()
        dsrc = K.gather_rows(dy, pos32)
        dx = dy
        if ctx.replace:
            dx = dy.clone()
            K.scatter_rows_(dx, pos32, torch.zeros_like(dsrc), True)
        return dx, None, dsrc, None


def first_true_rows(mask, n: int):
    """Positions of the first ``n`` true entries of a 1-D bool mask, in order, without a host
    synchronisation (a stable sort instead of ``nonzero``), and a bool [len, 1] that is false
    where the mask has fewer than that many true entries (those positions are arbitrary)."""
    n = min(int(n), mask.numel())
    pos = torch.argsort((~mask).to(torch.uint8), stable=True)[:n]
    return pos, mask.index_select(0, pos).unsqueeze(-1)


def scatter_rows(x, pos, src, replace: bool = False):
    """x with rows ``pos`` (unique) replaced by / increased by the rows of ``src``."""
    if use_kernels(x) and x.dim() == 2 and x.shape[1] % 8 == 0 and src.dtype == x.dtype:
        return _ScatterRowsFn.apply(x.contiguous(), pos.to(torch.int32), src.contiguous(), bool(replace))
    if replace:
        keep = torch.ones(x.shape[0], 1, dtype=x.dtype, device=x.device).index_fill(0, pos, 0.0)
        x = x * keep
    return x.index_add(0, pos, src.to(x.dtype))


class _Gather4Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, idx, w):
        ctx.save_for_backward(idx, w)
        ctx.t_ref, ctx.shape = table, table.shape
        return K.gather4_fwd(table, idx, w)

    @staticmethod
    def backward(ctx, dout):
        idx, w = ctx.saved_tensors
        mg = getattr(ctx.t_ref, "main_grad", None)
        dt = mg if mg is not None else torch.zeros(ctx.shape, dtype=torch.float32, device=dout.device)
        K.gather4_bwd(dout.contiguous(), idx, w, dt)
        return (None if mg is not None else dt.to(ctx.t_ref.dtype)), None, None


def gather4(table, idx_N4, w_N4):
    """out[i] = sum_k w[i,k] * table[idx[i,k]] (four-neighbour interpolation of a learned table)."""
    if use_kernels(table) and table.shape[1] % 8 == 0:
        return _Gather4Fn.apply(table, idx_N4.to(torch.int32).contiguous(), w_N4.float().contiguous())
    return (table[idx_N4.reshape(-1).long()].view(idx_N4.shape[0], 4, -1).float() * w_N4.float().unsqueeze(-1)).sum(1).to(table.dtype)


# ----------------------------------------------------------------------------- swiglu
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return K.swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dact):
        (gu,) = ctx.saved_tensors
        return K.swiglu_bwd(gu, dact)


def swiglu(gu):
    """gu = [gate | up] on the last dim -> silu(gate) * up."""
    if use_kernels(gu) and gu.shape[-1] % 16 == 0:
        return _SwiGLUFn.apply(gu.contiguous())
    return R.swiglu(gu)


class _SwiGLULinearFn(torch.autograd.Function):
    """y = (silu(gate) * up) @ w.T (+ residual) as one node.  Only [gate | up] is kept for the
    backward pass: the activation, which the weight gradient needs, comes back out of the SwiGLU
    backward kernel, which reads gate and up anyway.  When the output is already known (a layer
    re-run whose result nobody reads) nothing at all is computed in forward.  The backward pass is
    the last reader of [gate | up] and writes its gradient over it (a non-leaf input only; a graph
    kept for a second backward pass would find it overwritten)."""

    @staticmethod
    def forward(ctx, gu, w, residual, y_pre=None):
        shp = gu.shape
        g2 = gu.reshape(-1, shp[-1])
        y = y_pre
        if y is None:
            y = K.gemm(K.swiglu_fwd(g2), w, residual=residual)
        ctx.save_for_backward(g2, w)
        ctx.shp = shp
        ctx.has_res = residual is not None
        ctx.w_ref = w
        ctx.inplace = bool(gu.requires_grad and not gu.is_leaf and g2.is_contiguous())
        return y.view(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        g2, w = ctx.saved_tensors
        w_obj = ctx.w_ref
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dact = K.gemm(dy2, w, b_mn=True)
        dgu, act = K.swiglu_bwd(g2, dact, with_act=True, inplace=ctx.inplace)
        del dact
        dw = None
        pg = getattr(w_obj, "peer_grad", None)
        if ctx.needs_input_grad[1] and pg is not None:
            K.gemm_peer_reduce(dy2, act, pg[0], pg[1], pg[2], a_mn=True, b_mn=True)
        elif ctx.needs_input_grad[1]:
            dw = _acc_main_grad(
                w_obj,
                lambda mg: K.gemm(dy2, act, a_mn=True, b_mn=True, out=mg, accumulate=True),
                lambda: K.gemm(dy2, act, a_mn=True, b_mn=True),
            )
        return dgu.view(ctx.shp), dw, (dy if ctx.has_res else None), None


def swiglu_linear(gu, w, residual=None, tag=None):
    """linear(swiglu(gu), w, residual) -- the second half of a SwiGLU feed-forward block."""
    if (use_kernels(gu) and w.dtype == bf16 and gu.shape[-1] % 16 == 0 and w.shape[0] % 8 == 0
            and getattr(w, "ag_spec", None) is None):
        key, pre = _stash_lookup(tag)
        if pre is _SKIP:
            pre = torch.empty(gu.numel() // gu.shape[-1], w.shape[0], dtype=gu.dtype, device=gu.device)
        y = _SwiGLULinearFn.apply(gu.contiguous(), w, residual, None if pre is None else pre.view(-1, w.shape[0]))
        _stash_store(key, y)
        return y
    return linear(swiglu(gu), w, residual, tag=tag)


# ----------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        ctx.save_for_backward(ids)
        ctx.t_ref = table
        return K.embedding_fwd(ids, table)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        t = ctx.t_ref
        pg = getattr(t, "peer_embed_grad", None)
        if pg is not None:      # table rows sharded over the GPUs: rows go to their owners over NVLink
            K.embedding_bwd_peer(ids, dy, pg[0], pg[1])
            return None, None
        mg = getattr(t, "main_grad", None)
        if mg is not None:
            K.embedding_bwd(ids, dy, mg)
            return None, None
        g = torch.zeros(t.shape, dtype=torch.float32, device=t.device)
        K.embedding_bwd(ids, dy, g)
        return None, g.to(t.dtype)


def embedding(ids, table):
    if table.is_cuda and table.dtype == bf16 and use_kernels(table) and table.shape[1] % 8 == 0:
        return _EmbeddingFn.apply(ids, table)
    return torch.nn.functional.embedding(ids.long(), table)


# ----------------------------------------------------------------------------- qk-norm + rope
class _QKNormRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, qw, kw, cos, sin, H, G, Kd, rot, eps, one_plus, q_stride_heads):
        q, k = K.qknorm_rope_fwd(qkv, qw, kw, cos, sin, H, G, Kd, rot, eps, one_plus, q_stride_heads)
        ctx.save_for_backward(qkv, qw, kw, cos, sin)
        ctx.cfg = (H, G, Kd, rot, eps, one_plus, q_stride_heads)
        ctx.qw_ref, ctx.kw_ref = qw, kw
        return q, k

    @staticmethod
    def backward(ctx, dq, dk):
        qkv, qw, kw, cos, sin = ctx.saved_tensors
        H, G, Kd, rot, eps, one_plus, qs = ctx.cfg
        dqkv = torch.zeros_like(qkv) if qs != 1 else torch.empty_like(qkv)
        if qs == 1:
            dqkv.view(qkv.shape[0], H + 2 * G, Kd)[:, H + G:].zero_()
        dqw = dkw = None
        qmg = getattr(ctx.qw_ref, "main_grad", None) if qw is not None else None
        kmg = getattr(ctx.kw_ref, "main_grad", None) if kw is not None else None
        if qw is not None:
            dqw_buf = qmg if qmg is not None else torch.zeros(Kd, dtype=torch.float32, device=qkv.device)
            dkw_buf = kmg if kmg is not None else torch.zeros(Kd, dtype=torch.float32, device=qkv.device)
        else:
            dqw_buf = dkw_buf = None
        K.qknorm_rope_bwd(qkv, qw, kw, cos, sin, dq.contiguous(), dk.contiguous(), dqkv, dqw_buf,
                          dkw_buf, H, G, Kd, rot, eps, one_plus, qs)
        if qw is not None and qmg is None:
            dqw = dqw_buf.to(qw.dtype)
        if kw is not None and kmg is None:
            dkw = dkw_buf.to(kw.dtype)
        return dqkv, dqw, dkw, None, None, None, None, None, None, None, None, None


def qk_norm_rope(qkv, qw, kw, sin, cos, H: int, G: int, Kd: int, rot: int | None = None,
                 eps: float = 1e-6, one_plus: bool = False, q_stride_heads: int = 1,
                 scale_in_dtype: bool = False):
    """Split a fused projection [M, (H*q_stride_heads + 2G) * Kd] into q, k, v; apply the
    per-head RMSNorm (weights may be None) and rotate-half RoPE on the first ``rot`` channels.

    sin/cos: fp32 [M, rot/2].  With ``q_stride_heads == 2`` every q head is followed by a
    gate head of the same width (gated attention); the gates are returned as a 4th value.
    Returns q [M,H,Kd], k [M,G,Kd], v [M,G,Kd] (a strided view), gate or None.
    """
    rot = Kd if rot is None else rot
    M = qkv.shape[0]
    qw_total = H * Kd * q_stride_heads
    v = qkv[:, qw_total + G * Kd:].view(M, G, Kd)
    gate = None
    if q_stride_heads == 2:
        gate = qkv[:, :qw_total].view(M, H, 2, Kd)[:, :, 1]
    if use_kernels(qkv) and (qw is None or qw.dtype == bf16):
        q, k = _QKNormRopeFn.apply(qkv, qw, kw, cos.contiguous(), sin.contiguous(), H, G, Kd, rot,
                                   eps, one_plus, q_stride_heads)
        return q, k, v, gate
    if q_stride_heads == 2:
        q = qkv[:, :qw_total].view(M, H, 2, Kd)[:, :, 0]
    else:
        q = qkv[:, :qw_total].view(M, H, Kd)
    k = qkv[:, qw_total:qw_total + G * Kd].view(M, G, Kd)
    if qw is not None:
        q = R.rmsnorm(q, qw, eps, one_plus, scale_in_dtype)
        k = R.rmsnorm(k, kw, eps, one_plus, scale_in_dtype)
    q = R.apply_rope(q, sin, cos, rot)
    k = R.apply_rope(k, sin, cos, rot)
    return q, k, v, gate


# ----------------------------------------------------------------------------- sigmoid output gate
class _SigmoidGateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o, gate):
        ctx.save_for_backward(o, gate)
        return K.sigmoid_gate_fwd(o, gate)

    @staticmethod
    def backward(ctx, dout):
        o, gate = ctx.saved_tensors
        return K.sigmoid_gate_bwd(o, gate, dout.contiguous())


def sigmoid_gate(o, gate):
    """o * sigmoid(gate) (output gate of the Qwen3.5 attention, reference
    omegalax/models/qwen3_5/attention.py:122); ``gate`` may be a strided view of the fused projection."""
    if use_kernels(o) and o.dim() == 3 and o.is_contiguous() and gate.dtype == bf16 and gate.stride(2) == 1 \
            and o.shape[2] % 8 == 0 and gate.stride(0) % 8 == 0 and gate.stride(1) % 8 == 0:
        return _SigmoidGateFn.apply(o, gate)
    return o * torch.sigmoid(gate.to(o.dtype))


# ----------------------------------------------------------------------------- attention
_ATTN_BWD_IMPL = {"impl": None}


def _attn_bwd_dispatch(q, k, v, o, lse, do, cu_seqlens, max_seqlen, scale, causal):
    """dq, dk, dv of packed-row attention."""
    if q.shape[-1] in (128, 256) and os.environ.get("OMEGALAX_B200_ATTN_BWD", "sm100") == "sm100":
        return K.attn_bwd(q, k, v, o, lse, do, cu_seqlens, max_seqlen, scale, causal)
    if q.shape[-1] == 64 and os.environ.get("OMEGALAX_B200_ATTN_BWD", "sm100") == "sm100":
        # 64-wide heads (vision tower): run the 128-wide kernel on zero-padded heads.  The padding
        # channels add nothing to q.k and receive zero gradients; the scale stays that of width 64.
        pad = lambda t: F.pad(t, (0, 64))
        dq, dk, dv = K.attn_bwd(pad(q), pad(k), pad(v), pad(o), lse, pad(do), cu_seqlens, max_seqlen, scale, causal)
        return dq[..., :64].contiguous(), dk[..., :64].contiguous(), dv[..., :64].contiguous()
    # recompute through the PyTorch definition (reference quality; used only until the
    # tcgen05 backward is selected)
    with torch.enable_grad():
        qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
        N, H, Kd = q.shape
        G = k.shape[1]
        B = cu_seqlens.numel() - 1
        if N == B * max_seqlen:
            out = torch.nn.functional.scaled_dot_product_attention(
                qq.view(B, max_seqlen, H, Kd).transpose(1, 2),
                kk.reshape(B, max_seqlen, G, Kd).transpose(1, 2),
                vv.reshape(B, max_seqlen, G, Kd).transpose(1, 2),
                is_causal=bool(causal), scale=scale, enable_gqa=True,
            ).transpose(1, 2).reshape(N, H, Kd)
        else:
            out = R.attention_varlen(qq, kk, vv, cu_seqlens, causal=bool(causal), scale=scale)
        return torch.autograd.grad(out, (qq, kk, vv), do)


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, scale, causal, pre=None):
        if pre is not None:
            o, lse = pre
        else:
            o, lse = K.attn_fwd(q, k, v, cu_seqlens, max_seqlen, scale, causal)
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens)
        ctx.cfg = (max_seqlen, scale, causal)
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse, cu = ctx.saved_tensors
        max_seqlen, scale, causal = ctx.cfg
        dq, dk, dv = _attn_bwd_dispatch(q, k, v, o, lse, do.contiguous(), cu, max_seqlen, scale, causal)
        return dq, dk, dv, None, None, None, None, None


def flash_attention(q, k, v, cu_seqlens, max_seqlen: int, *, scale: float, causal: bool, tag=None):
    """Packed-row attention.  q [N,H,Kd]; k, v [N,G,Kd]; cu_seqlens int32 [B+1]."""
    if use_kernels(q) and q.shape[-1] in (64, 128, 256):
        key, pre = _stash_lookup(tag)
        o, lse = _FlashAttnFn.apply(q, k, v, cu_seqlens, int(max_seqlen), float(scale), bool(causal), pre)
        _stash_store(key, (o, lse))
        return o
    if library_mode() and q.is_cuda:
        return _sdpa_packed(q, k, v, cu_seqlens, int(max_seqlen), float(scale), bool(causal))
    return R.attention_varlen(q, k, v, cu_seqlens, causal=causal, scale=scale)


# ----------------------------------------------------------------------------- linear + CE
class _LinearCEFn(torch.autograd.Function):
    """loss = grad-ready fused  sum_rows mask * nll(h W^T) * scale.

    Per row chunk: the logits GEMM keeps the fp32 accumulator's softmax statistics (maximum and sum
    of exponentials per 256-column tile, the target's logit) in its epilogue, so the loss and the
    log-sum-exp are those of fp32 logits, as in the reference (omegalax/trainers/loss.py:24-35); the
    bf16 copy of the chunk's logits that it also writes is turned into dlogits in place and feeds
    the dH and dW GEMMs of the same sweep.  No [B,T,V] tensor exists and the backward only
    rescales; dW goes straight into ``w.main_grad`` when it exists.  (Keeping dlogits out of
    memory altogether would need the [chunk, D] dH accumulator in TMEM, 4096 columns against the
    512 there are, or a third pass of the logits GEMM, which costs more than the traffic saved.)
    """

    @staticmethod
    def forward(ctx, h, w, targets, mask, scale_t, chunk):
        M, D = h.shape
        V = w.shape[0]
        dev = h.device
        loss_sum = torch.zeros(1, dtype=torch.float32, device=dev)
        need_grad = h.requires_grad or w.requires_grad
        mg = getattr(w, "main_grad", None)
        pg = getattr(w, "peer_grad", None)
        dh = torch.empty_like(h) if need_grad else None
        dw = None
        if need_grad and w.requires_grad and pg is None:
            dw = mg if mg is not None else torch.zeros(V, D, dtype=torch.float32, device=dev)
        t32 = targets.to(torch.int32).contiguous()
        mk = mask.to(torch.float32).contiguous()
        logits = torch.empty(min(chunk, M), V, dtype=bf16, device=dev)
        n_tiles = -(-V // 256)
        stats = torch.empty(min(chunk, M), n_tiles, 2, dtype=torch.float32, device=dev)
        tgt_logit = torch.zeros(min(chunk, M), dtype=torch.float32, device=dev)
        lse = torch.empty(min(chunk, M), dtype=torch.float32, device=dev)
        fp32_stats = os.environ.get("OMEGALAX_B200_CE_STATS", "1") == "1" and h.shape[1] % 8 == 0
        for r0 in range(0, M, chunk):
            r1 = min(M, r0 + chunk)
            lg = logits[: r1 - r0]
            hc = h[r0:r1]
            if fp32_stats:
                n = r1 - r0
                K.gemm(hc, w, out=lg, ce=(t32[r0:r1], stats[:n], tgt_logit[:n]))
                K.ce_finish(stats[:n], tgt_logit[:n], mk[r0:r1], loss_sum, lse[:n])
                if need_grad:
                    K.ce_vp_grad_(lg, t32[r0:r1], 0, lse[:n], mk[r0:r1], scale_t)
            else:
                K.gemm(hc, w, out=lg)
                K.ce_fwd_bwd(lg, t32[r0:r1], mk[r0:r1], scale_t, loss_sum, write_grad=need_grad)
            if need_grad:
                K.gemm(lg, w, b_mn=True, out=dh[r0:r1])
                if pg is not None:
                    K.gemm_peer_reduce(lg, hc, pg[0], pg[1], pg[2], a_mn=True, b_mn=True)
                elif dw is not None:
                    K.gemm(lg, hc, a_mn=True, b_mn=True, out=dw, accumulate=True)
        ctx.save_for_backward(dh)
        ctx.dw = None if (mg is not None or dw is None) else dw
        ctx.w_dtype = w.dtype
        return (loss_sum * scale_t).squeeze(0)

    @staticmethod
    def backward(ctx, g):
        (dh,) = ctx.saved_tensors
        dw = ctx.dw
        gh = None if dh is None else (dh * g.to(dh.dtype))
        gw = None if dw is None else (dw * g).to(ctx.w_dtype)
        return gh, gw, None, None, None, None


class _VocabParallelCEFn(torch.autograd.Function):
    """Cross-entropy with the head split over the tensor-parallel ranks on the vocabulary and
    the hidden rows split on the sequence.  h [M/tp, D] (this rank's rows), w [V/tp, D] (this
    rank's vocabulary slice), targets / mask [M] for all rows.  The rows are gathered, every rank
    scores them against its slice, the per-row (max, sum-exp, target logit) are combined with
    two small all-reduces, and the gradients are produced in the same sweep: dW stays local,
    the partial dH of the slices is reduce-scattered back to the row owners.  The returned loss
    is 1/tp of the full loss (the ranks' values add up to it); the stored gradients are those
    of the full loss."""

    @staticmethod
    def forward(ctx, h, w, targets, mask, scale_t, tp, chunk):
        import torch.distributed as dist

        from ..parallel import tp as tp_lib

        use_k = use_kernels(h) and w.dtype == bf16
        h_full = tp_lib._ag_rows(h.contiguous(), tp)
        M, D = h_full.shape
        Vl = w.shape[0]
        v0 = tp.rank * Vl
        dev = h.device
        need_grad = h.requires_grad or w.requires_grad
        mg = getattr(w, "main_grad", None)
        pg = getattr(w, "peer_grad", None)
        dh_full = torch.empty_like(h_full) if need_grad else None
        dw = None
        if need_grad and w.requires_grad and pg is None:
            dw = mg if mg is not None else torch.zeros(Vl, D, dtype=torch.float32, device=dev)
        t32 = targets.to(torch.int32).contiguous()
        mk = mask.to(torch.float32).contiguous()
        loss_sum = torch.zeros(1, dtype=torch.float32, device=dev)
        for r0 in range(0, M, chunk):
            r1 = min(M, r0 + chunk)
            hc = h_full[r0:r1]
            if use_k:
                lg = K.gemm(hc, w)
                mx, sm, tg = K.ce_vp_stats(lg, t32[r0:r1], v0)
            else:
                lg = (hc.float() @ w.float().t())
                mx = lg.max(-1).values
                sm = torch.exp(lg - mx[:, None]).sum(-1)
                loc = t32[r0:r1].long() - v0
                ok = (loc >= 0) & (loc < Vl)
                tg = torch.where(ok, lg.gather(1, loc.clamp(0, Vl - 1)[:, None]).squeeze(1), torch.zeros_like(mx))
            gmax = mx.clone()
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=tp.group)
            pack = torch.stack([sm * torch.exp(mx - gmax), tg])
            dist.all_reduce(pack, group=tp.group)
            lse = gmax + torch.log(pack[0])
            loss_sum += (mk[r0:r1] * (lse - pack[1])).sum()
            if not need_grad:
                continue
            if use_k:
                K.ce_vp_grad_(lg, t32[r0:r1], v0, lse.contiguous(), mk[r0:r1], scale_t)
                K.gemm(lg, w, b_mn=True, out=dh_full[r0:r1])
                if pg is not None:
                    K.gemm_peer_reduce(lg, hc, pg[0], pg[1], pg[2], a_mn=True, b_mn=True)
                elif dw is not None:
                    K.gemm(lg, hc, a_mn=True, b_mn=True, out=dw, accumulate=True)
            else:
                p_ = torch.exp(lg - lse[:, None])
                loc = t32[r0:r1].long() - v0
                ok = (loc >= 0) & (loc < Vl)
                p_[ok.nonzero().squeeze(1), loc[ok]] -= 1.0
                dl = p_ * (mk[r0:r1] * scale_t)[:, None]
                dh_full[r0:r1] = (dl @ w.float()).to(h.dtype)
                if dw is not None:
                    dw += dl.t() @ hc.float()
        dh = tp_lib._rs_rows(dh_full, tp) if need_grad else None
        ctx.save_for_backward(dh)
        ctx.dw = None if (mg is not None or dw is None) else dw
        ctx.w_dtype = w.dtype
        return (loss_sum * scale_t).squeeze(0) / tp.size

    @staticmethod
    def backward(ctx, g):
        (dh,) = ctx.saved_tensors
        dw = ctx.dw
        gh = None if dh is None else (dh * g.to(dh.dtype))
        gw = None if dw is None else (dw * g).to(ctx.w_dtype)
        return gh, gw, None, None, None, None, None


def linear_cross_entropy_vocab_parallel(h_local, w_local, targets, mask, scale, tp, chunk: int = 4096):
    """Vocabulary-parallel fused linear + cross-entropy (see ``_VocabParallelCEFn``)."""
    if not torch.is_tensor(scale):
        scale = torch.tensor([float(scale)], dtype=torch.float32, device=h_local.device)
    return _VocabParallelCEFn.apply(h_local, w_local, targets, mask, scale.reshape(1).to(torch.float32), tp, chunk)


def linear_cross_entropy(h, w, targets, mask, scale, chunk: int = 4096):
    """scale * sum_i mask_i * CE(h_i W^T, targets_i).

    h [M,D], w [V,D], targets [M] int, mask [M]; ``scale`` is a float or a 1-element fp32
    tensor (e.g. 1 / number of supervised tokens, computed on the device).  On the kernel
    path the gradient is produced during the forward sweep and assumes this loss is
    differentiated with an upstream gradient of one when ``w.main_grad`` is in use.
    """
    if not torch.is_tensor(scale):
        scale = torch.tensor([float(scale)], dtype=torch.float32, device=h.device)
    scale = scale.reshape(1).to(torch.float32)
    if use_kernels(h) and w.dtype == bf16 and w.shape[0] % 8 == 0:
        return _LinearCEFn.apply(h.contiguous(), w, targets, mask, scale, chunk)
    total = h.new_zeros((), dtype=torch.float32)
    ckpt = library_mode() and torch.is_grad_enabled() and (h.requires_grad or w.requires_grad)
    for r0 in range(0, h.shape[0], chunk):
        r1 = min(h.shape[0], r0 + chunk)
        if ckpt:   # the usual memory-saving recipe: the chunk's logits are recomputed in the backward
            from torch.utils.checkpoint import checkpoint

            total = total + checkpoint(R.cross_entropy_sum, h[r0:r1], w, targets[r0:r1], mask[r0:r1],
                                       use_reentrant=False)
        else:
            total = total + R.cross_entropy_sum(h[r0:r1], w, targets[r0:r1], mask[r0:r1])
    return total * scale.squeeze(0)


# ----------------------------------------------------------------------------- GatedDeltaNet ops
class _CausalConv1dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        ctx.w_ref = w
        return K.causal_conv1d_fwd(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        mg = getattr(ctx.w_ref, "main_grad", None)
        dwf = mg if mg is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        dx = K.causal_conv1d_bwd(x, w, dy.contiguous(), dwf)
        return dx, (None if mg is not None else dwf.to(w.dtype))


def causal_conv1d_silu(x_BTC, w_CK):
    """Depthwise causal conv over time (left pad K-1) followed by SiLU.  x [B,T,C], w [C,K]."""
    if use_kernels(x_BTC) and w_CK.dtype == bf16 and w_CK.shape[1] == 4 and x_BTC.shape[-1] % 8 == 0:
        return _CausalConv1dFn.apply(x_BTC.contiguous(), w_CK.contiguous())
    y = R.causal_conv1d(x_BTC.transpose(1, 2), w_CK, activation_silu=True)
    return y.transpose(1, 2)


class _GatedDeltaRuleFn(torch.autograd.Function):
    """fp32 tensors, T a multiple of 64; q,k already normalised / scaled."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, s0, want_final):
        save = any(ctx.needs_input_grad[:6])
        o, n_out, states, s_final = K.gdn_fwd(q, k, v, g, beta, s0=s0, save=save, want_final=want_final)
        if save:
            ctx.save_for_backward(q, k, v, g, beta, n_out, states)
        ctx.has_s0 = s0 is not None
        if want_final:
            return o, s_final
        return o, None

    @staticmethod
    def backward(ctx, d_o, d_sf):
        q, k, v, g, beta, n_out, states = ctx.saved_tensors
        dq, dk, dv, dg, dbeta, ds0 = K.gdn_bwd(q, k, v, g, beta, n_out, states, d_o.contiguous(),
                                               d_sfinal=None if d_sf is None else d_sf.contiguous(),
                                               want_ds0=ctx.has_s0)
        return dq, dk, dv, dg, dbeta, ds0, None


def gated_delta_rule(q, k, v, g, beta, chunk: int = 64, initial_state=None, output_final_state=False):
    """Chunked gated delta rule (fp32 inside); q,k [B,T,Hk,A] with Hk dividing H, v [B,T,H,U],
    g/beta [B,T,H].  Key heads are shared by groups of H/Hk value heads."""
    H, Hk = v.shape[2], q.shape[2]
    if use_kernels(v) and q.shape[-1] == 128 and v.shape[-1] % 64 == 0 and chunk == 64:
        dt, T, A = v.dtype, q.shape[1], q.shape[-1]
        qf = R.l2norm(q.float()) * (A ** -0.5)
        kf = R.l2norm(k.float())
        vf, gf, bf_ = v.float(), g.float(), beta.float()
        pad = (-T) % 64
        if pad:
            qf, kf, vf = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (qf, kf, vf))
            gf, bf_ = (F.pad(t, (0, 0, 0, pad)) for t in (gf, bf_))
        s0 = None if initial_state is None else initial_state.float().contiguous()
        o, sf = _GatedDeltaRuleFn.apply(qf.contiguous(), kf.contiguous(), vf.contiguous(), gf.contiguous(),
                                        bf_.contiguous(), s0, output_final_state)
        o = o[:, :T].to(dt)
        return (o, sf) if output_final_state else o
    if Hk != H:
        q = q.repeat_interleave(H // Hk, dim=2)
        k = k.repeat_interleave(H // Hk, dim=2)
    return R.chunk_gated_delta_rule(q, k, v, g, beta, chunk=chunk, initial_state=initial_state,
                                    output_final_state=output_final_state)