"""Token-choice mixture-of-experts: routing, permutation, grouped expert MLP, combine.

Only the k selected experts of every token are evaluated (the reference evaluates every
expert for every token and then gathers, omegalax/models/qwen3/model.py:92-118; the
selected-expert math is identical).  On CUDA bf16 the expert MLPs run on the grouped
tcgen05 GEMM over rows permuted into per-expert segments padded to multiples of 128.
"""
from __future__ import annotations

import torch

from . import functional as Fn
from . import kernels as K
from . import reference as R

bf16 = torch.bfloat16
# Expert segments are padded to multiples of PAD rows.  256 lets the grouped GEMMs run on CTA pairs
# (a 256-row pair tile must lie inside one expert's segment); OMEGALAX_B200_MOE_PAD=128 selects the
# single-CTA grouped kernel and its smaller padding.
import os as _os

PAD = int(_os.environ.get("OMEGALAX_B200_MOE_PAD", "256"))
_PAIR = PAD % 256 == 0


class _RouteFn(torch.autograd.Function):
    """Router kernel: softmax + top-k + renormalisation in one pass, analytic backward."""

    @staticmethod
    def forward(ctx, logits, top_k, renormalize):
        probs, w, idx32 = K.router_topk(logits, top_k, renormalize)
        ctx.save_for_backward(probs, w, idx32)
        ctx.renorm = renormalize
        ctx.set_materialize_grads(False)
        idx = idx32.to(torch.int64)
        ctx.mark_non_differentiable(idx)
        return probs, w, idx

    @staticmethod
    def backward(ctx, dprobs, dw, _didx):
        probs, w, idx32 = ctx.saved_tensors
        if dw is None:
            dw = torch.zeros_like(w)
        dp = None if dprobs is None else dprobs.contiguous().float()
        return K.router_topk_bwd(probs, w, idx32, dw.contiguous().float(), dp, ctx.renorm), None, None


def route(router_logits, top_k: int, renormalize: bool):
    """fp32 softmax over experts, top-k, optional renormalisation with clip(sum, 1e-9).
    Returns probs [M,E] fp32, weights [M,k] fp32, indices [M,k] int64."""
    E = router_logits.shape[-1]
    if Fn.use_kernels(router_logits) and router_logits.dtype == bf16 and router_logits.dim() == 2 \
            and E % 32 == 0 and E <= 512 and top_k <= 16:
        return _RouteFn.apply(router_logits.contiguous(), top_k, bool(renormalize))
    probs = torch.softmax(router_logits.float(), dim=-1)
    # stable sort: equal probabilities (frequent with bf16 logits) go to the lower expert id, the
    # same rule as the router kernel
    w, idx = torch.sort(probs, dim=-1, descending=True, stable=True)
    w, idx = w[..., :top_k], idx[..., :top_k]
    if renormalize:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-9)
    return probs, w, idx


def _global_sum(local, group):
    """Sum of ``local`` over the data ranks of ``group``.  The value is the global sum on every
    rank; the derivative with respect to this rank's ``local`` is W (the group size), so that a
    caller that adds loss/W on each of the W ranks -- gradients are summed over ranks -- ends up
    with exactly the gradient of the global loss."""
    import torch.distributed as dist

    W = dist.get_world_size(group)
    tot = local.detach().clone()
    dist.all_reduce(tot, group=group)
    return W * local + (tot - W * local.detach()), W


def load_balance_loss_qwen3(probs, idx, num_experts: int, coef: float, group=None):
    """coef * E * sum_e (fraction of (token,slot) picks of e per token) * mean prob of e,
    over all tokens including padding (omegalax/models/qwen3/model.py:120-124).  With ``group``
    the two statistics are taken over the tokens of every data rank (one all-reduce of 2E
    floats), which is what the reference computes under SPMD over the global batch."""
    M = probs.shape[0]
    counts = torch.zeros(num_experts, dtype=torch.float32, device=probs.device)
    counts.scatter_add_(0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.float32, device=probs.device))
    if group is None or coef == 0.0:
        return coef * num_experts * torch.sum((counts / M) * probs.mean(0))
    stats, W = _global_sum(torch.cat([counts, probs.float().sum(0)]), group)
    counts_g, psum_g = stats[:num_experts].detach(), stats[num_experts:]
    return coef * num_experts * torch.sum((counts_g / (M * W)) * (psum_g / (M * W)))


def load_balance_loss_sq(probs, num_experts: int, coef: float, group=None):
    """coef * sum_e (mean prob of e - 1/E)^2 (omegalax/models/qwen3_5/model.py:172-174); with
    ``group`` the mean is over the tokens of every data rank."""
    if group is None or coef == 0.0:
        return coef * torch.sum((probs.mean(0) - 1.0 / num_experts) ** 2)
    psum_g, W = _global_sum(probs.float().sum(0), group)
    return coef * torch.sum((psum_g / (probs.shape[0] * W) - 1.0 / num_experts) ** 2)


def build_permutation(idx, num_experts: int, pad: int = PAD):
    """Sort (token, slot) pairs by expert into segments padded to multiples of ``pad``.

    Returns
      dest      [M*k] int64 : row of the padded buffer that pair p = token*k + slot goes to
      offsets   [E+1] int32 : segment boundaries (multiples of pad)
      capacity  int         : static row count of the padded buffer
    No host synchronisation: the capacity is the worst case M*k + E*(pad-1) rounded up.
    """
    Mk = idx.numel()
    flat = idx.reshape(-1)
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + pad - 1) // pad * pad
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=idx.device)
    offsets[1:] = padded.cumsum(0)
    order = torch.argsort(flat, stable=True)
    starts_unpadded = counts.cumsum(0) - counts
    sorted_e = flat[order]
    rank_in_e = torch.arange(Mk, device=idx.device) - starts_unpadded[sorted_e]
    dest_sorted = offsets[sorted_e] + rank_in_e
    dest = torch.empty_like(dest_sorted)
    dest[order] = dest_sorted
    capacity = (Mk + num_experts * (pad - 1) + pad - 1) // pad * pad
    return dest, offsets.to(torch.int32), capacity


class _GroupedLinearFn(torch.autograd.Function):
    """y[rows of e] = x[rows of e] @ w[e].T for w [E,N,K]."""

    @staticmethod
    def forward(ctx, x, w, offsets, out=None):
        y = K.gemm_grouped(x, w, offsets, out=out, pair=_PAIR)
        ctx.save_for_backward(x, w, offsets)
        ctx.w_ref = w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, offsets = ctx.saved_tensors
        dy = dy.contiguous()
        dx = K.gemm_grouped(dy, w, offsets, b_mn=True, pair=_PAIR) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                K.gemm_grouped_wgrad(dy, x, offsets, mg, accumulate=True, pair=_PAIR)
            else:
                dwf = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
                K.gemm_grouped_wgrad(dy, x, offsets, dwf, accumulate=False, pair=_PAIR)
                dw = dwf.to(w.dtype)
        return dx, dw, None, None


def grouped_linear(x, w, offsets, out=None):
    return _GroupedLinearFn.apply(x, w, offsets, out)


def expert_mlp_permuted(xp, w_gate_up, w_down, offsets, out=None):
    """SwiGLU expert MLP on rows already grouped by expert (padded layout).  ``out`` may name
    the buffer that receives the result (e.g. the exchange buffer the combine step reads)."""
    gu = grouped_linear(xp, w_gate_up, offsets)
    act = Fn.swiglu(gu)
    return grouped_linear(act, w_down, offsets, out)


# ---- row movement on one GPU: the dispatch / combine kernels of the expert-parallel path with a
# single "rank" whose buffer is a local tensor
def _ptr1(t):
    import ctypes

    return (ctypes.c_void_p * 1)(t.data_ptr())


def _push_rows(buf, src, src_tok, rank0, dst_row, scale):
    from . import lib

    lib.call("ob_ep_push", _ptr1(buf), 1, src.data_ptr(), src_tok.data_ptr(), rank0.data_ptr(), dst_row.data_ptr(),
             lib.ptr(scale), dst_row.numel(), src.shape[1], lib.stream_ptr())


def _pull_rows(buf, rank0, src_row, M, k, weights=None, want_out=True, grad=None):
    from . import lib

    D = buf.shape[1]
    out = torch.empty(M, D, dtype=buf.dtype, device=buf.device) if want_out else None
    dots = torch.empty(M * k, dtype=torch.float32, device=buf.device) if grad is not None else None
    lib.call("ob_ep_pull", _ptr1(buf), 1, lib.ptr(out), rank0.data_ptr(), src_row.data_ptr(), lib.ptr(weights),
             lib.ptr(grad), lib.ptr(dots), M, k, D, lib.stream_ptr())
    return out, dots


class _LocalDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dest, src_tok, rank0, cap, k):
        xp = torch.zeros(cap, x.shape[1], dtype=x.dtype, device=x.device)   # padding rows stay zero
        _push_rows(xp, x, src_tok, rank0, dest, None)
        ctx.save_for_backward(dest, rank0)
        ctx.M, ctx.k = x.shape[0], k
        return xp

    @staticmethod
    def backward(ctx, d_xp):
        dest, rank0 = ctx.saved_tensors
        dx, _ = _pull_rows(d_xp.contiguous(), rank0, dest, ctx.M, ctx.k)
        return dx, None, None, None, None, None


class _LocalCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, yp, weights, dest, src_tok, rank0):
        M, k = weights.shape
        y, _ = _pull_rows(yp, rank0, dest, M, k, weights=weights.reshape(-1))
        ctx.save_for_backward(yp, weights, dest, src_tok, rank0)
        return y

    @staticmethod
    def backward(ctx, dy):
        yp, weights, dest, src_tok, rank0 = ctx.saved_tensors
        M, k = weights.shape
        dy = dy.contiguous()
        _, dots = _pull_rows(yp, rank0, dest, M, k, want_out=False, grad=dy)
        d_yp = torch.zeros_like(yp)
        _push_rows(d_yp, dy, src_tok, rank0, dest, weights.reshape(-1))
        return d_yp, dots.view(M, k), None, None, None


def moe_mlp(x, weights, idx, w_gate_up, w_down):
    """Routed SwiGLU experts.  x [M,D]; weights/idx [M,k]; w_gate_up [E,2F,D] with rows
    [gate | up]; w_down [E,D,F].  Returns [M,D] = sum_k weights * expert_{idx}(x)."""
    M, D = x.shape
    E = w_gate_up.shape[0]
    k = idx.shape[1]
    if Fn.use_kernels(x) and w_gate_up.dtype == bf16 and D % 64 == 0:
        offsets, dest = K.moe_plan(idx.to(torch.int32).contiguous(), E, PAD)
        cap = (M * k + E * (PAD - 1) + PAD - 1) // PAD * PAD
        src_tok = torch.arange(M, device=x.device, dtype=torch.int32).repeat_interleave(k)
        rank0 = torch.zeros(M * k, dtype=torch.int32, device=x.device)
        xp = _LocalDispatch.apply(x.contiguous(), dest, src_tok, rank0, cap, k)
        yp = expert_mlp_permuted(xp, w_gate_up, w_down, offsets)
        return _LocalCombine.apply(yp, weights.contiguous().float(), dest, src_tok, rank0)
    out = torch.zeros(M, D, dtype=torch.float32, device=x.device)
    for e in range(E):
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x.index_select(0, tok)
        gu = xe @ w_gate_up[e].to(x.dtype).t()
        ye = R.swiglu(gu) @ w_down[e].to(x.dtype).t()
        out.index_add_(0, tok, ye.float() * weights[tok, slot].unsqueeze(-1))
    return out.to(x.dtype)
