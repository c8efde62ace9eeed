"""Tensor-level wrappers around the sm_100a launchers (no autograd here).

All functions take CUDA bf16 tensors unless noted, launch on the current stream and
return immediately.  ``launch_count`` counts every kernel of this library that was
launched since the last ``reset_launch_count()``.
"""
from __future__ import annotations

import os

import torch

from . import lib

bf16 = torch.bfloat16
_launches = 0


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def launch_count() -> int:
    return _launches


def _call(name, *args):
    global _launches
    _launches += 1
    lib.call(name, *args)


def _row_major_2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        t = t.reshape(-1, t.shape[-1])
    if t.stride(1) != 1 or (t.stride(0) % 8) or (t.data_ptr() % 16):
        t = t.contiguous()
    return t


_PAIR_MODE = os.environ.get("OMEGALAX_B200_GEMM_PAIR", "all")   # "0" never, "1" always, "all" / "auto" by shape


_PAIR_AG = os.environ.get("OMEGALAX_B200_GEMM_PAIR_AG", "1") == "1"   # gather mode on the pair kernel


def _use_pair(M: int, N: int, K: int, wgrad: bool = False) -> bool:
    """CTA-pair (256 x 256 tile) kernel for GEMMs with enough tiles to fill every SM pair."""
    if _PAIR_MODE == "0":
        return False
    if _PAIR_MODE == "1":
        return True
    big = (-(-M // 256)) * (-(-N // 256)) >= 74 and N >= 512 and K >= 256
    if _PAIR_MODE == "all":
        # Inside a training step (power-capped clocks) the pair kernel is the faster one on every
        # large GEMM: it needs about 10 % fewer SM cycles per step.
        return big
    # Timed alone in short bursts it wins on the attention-sized projections and loses on the
    # widest (MLP) ones and on weight gradients: "auto" keeps it to the former.
    return big and not wgrad and N <= 8192 and K <= 8192


def gemm(a, b, *, a_mn: bool = False, b_mn: bool = False, out=None, out_dtype=bf16,
         accumulate: bool = False, residual=None, bn: int = 0, pair: bool | None = None, bias=None,
         ce=None):
    """C = op(A) op(B)^T on the tcgen05 kernel.

    a: [M,K] (a_mn False) or [K,M] (a_mn True); b: [N,K] (b_mn False) or [K,N] (b_mn True).
    out: optional preallocated [M,N] (bf16 or fp32); ``accumulate`` adds into an fp32 out.
    ``bias`` (bf16 [N]) and ``residual`` (bf16 [M,N]) are added in the epilogue.  ``ce`` =
    (targets int32 [M], stats fp32 [M, ceil(N/256), 2], target_logit fp32 [M]) asks the 512 x 256
    tile kernel for the cross-entropy statistics of the fp32 accumulator (bf16 output only).
    """
    a = _row_major_2d(a)
    b = _row_major_2d(b)
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"reduction mismatch {K} vs {Kb}")
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    if out.stride(1) != 1:
        raise ValueError("out must be row-major")
    if out.dtype == bf16:
        mode = 0
        if accumulate:
            raise ValueError("accumulate needs an fp32 output")
    elif out.dtype == torch.float32:
        mode = 2 if accumulate else 1
    else:
        raise ValueError("out dtype must be bf16 or fp32")
    res_ptr, ldr = None, 0
    if residual is not None:
        residual = residual.reshape(M, N)
        if residual.stride(1) != 1:
            residual = residual.contiguous()
        res_ptr, ldr = residual.data_ptr(), residual.stride(0)
    st = lib.status_tensor(a.device)
    if bias is not None and (bias.dtype != bf16 or bias.numel() != N or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous bf16 vector of N elements")
    if pair is None:
        pair = bn == 0 and _use_pair(M, N, K, wgrad=a_mn and b_mn)
    if ce is not None:
        tg, stats, tl = ce
        if mode != 0 or residual is not None or tuple(stats.shape) != (M, -(-N // 256), 2) or tl.numel() != M:
            raise ValueError("cross-entropy statistics need a bf16 output, no residual and [M, ceil(N/256), 2] stats")
        pair = True
    if pair:
        ce_ptrs = (None, None, None) if ce is None else (ce[0].data_ptr(), ce[1].data_ptr(), ce[2].data_ptr())
        _call("ob_gemm_bf16_pair", a.data_ptr(), b.data_ptr(), out.data_ptr(), res_ptr, M, N, K,
              a.stride(0), b.stride(0), out.stride(0), ldr, int(a_mn), int(b_mn), mode, lib.ptr(bias), *ce_ptrs,
              st.data_ptr(), lib.stream_ptr())
        return out
    _call("ob_gemm_bf16", a.data_ptr(), b.data_ptr(), out.data_ptr(), res_ptr, M, N, K,
          a.stride(0), b.stride(0), out.stride(0), ldr, int(a_mn), int(b_mn), mode, bn, lib.ptr(bias),
          st.data_ptr(), lib.stream_ptr())
    return out


def gemm_peer_reduce(a, b, peer_ptrs, rows_per_peer: int, ldc: int, *, a_mn=False, b_mn=False, bf16_out=False,
                     pair: bool | None = None, slot: int | None = None):
    """GEMM whose result rows are added into buffers owned by other GPUs (``peer_ptrs[r]`` holds
    rows [r*rows_per_peer, (r+1)*rows_per_peer)): fp32 buffers by default (gradient shards), bf16
    buffers with ``bf16_out`` (activations: half the NVLink bytes, bf16 accumulation).  With
    ``slot`` nothing is reduced: the bf16 rows are stored into slab ``slot`` of the owner's staging
    buffer ([senders, rows_per_peer, ldc]) and the owner sums the slabs with ``slab_sum``.
    A ``peer_ptrs`` list with a ``rank`` attribute (``SymmetricBuffer.peer_ptr_list``) makes the
    tiles start with this GPU's own rows and walk the owners from there, so that the GPUs of the
    group write to distinct owners at any moment."""
    import ctypes

    a = _row_major_2d(a)
    b = _row_major_2d(b)
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N = b.shape[1] if b_mn else b.shape[0]
    arr = (ctypes.c_void_p * len(peer_ptrs))(*peer_ptrs)
    st = lib.status_tensor(a.device)
    if pair is None:
        pair = _use_pair(M, N, K, wgrad=a_mn and b_mn)
    name = "ob_gemm_bf16_pair_peer_reduce" if pair else "ob_gemm_bf16_peer_reduce"
    _call(name, a.data_ptr(), b.data_ptr(), ctypes.cast(arr, ctypes.c_void_p),
          len(peer_ptrs), rows_per_peer, M, N, K, a.stride(0), b.stride(0), ldc, int(a_mn),
          int(b_mn), (2 + int(slot)) if slot is not None else int(bf16_out), int(getattr(peer_ptrs, "rank", 0)),
          st.data_ptr(), lib.stream_ptr())


def slab_sum(staging, slots: int, out, residual=None):
    """out = sum of the ``slots`` equal slabs of ``staging`` (+ residual): bf16, fp32 accumulation."""
    _call("ob_slab_sum", staging.data_ptr(), int(slots), out.numel(), lib.ptr(residual), out.data_ptr(),
          lib.stream_ptr())
    return out


def ag_copy_ctas(M: int, N: int, Kd: int, total_bytes: float) -> int:
    """Copy CTAs for the gather mode.  The tiles walk the chunks in arrival order starting with this
    GPU's own chunk (read in place), so the chunks must arrive at the rate the tiles consume them:
    the whole operand within ~80 % of the GEMM's duration, at ~45 GB/s per copy thread (128 KB in
    flight)."""
    t_gemm = 2.0 * M * N * Kd / 1.1e15
    need = total_bytes / max(0.8 * t_gemm, 1e-6) / 45e9
    n = int(min(16, max(2, -(-need // 1))))
    return n + (n & 1)          # even: the CTA-pair kernel gives up whole clusters


def gemm_ag(other, full, src_ptrs, *, side: int, rank: int, rows_per_rank: int, flags, target: int,
            copy_ctas: int = 8, residual=None, out=None):
    """All-gather -> GEMM in one launch: y = A @ B^T with both operands [rows, K] row-major.
    side 1: A = ``full`` [rows_per_rank * W, K] is assembled from the ranks' row chunks at
    ``src_ptrs`` while the tiles run; side 2: B likewise.  ``other`` is the operand that is
    already complete.  ``flags`` (uint32 [W]) only grow: ``target`` is their value after this call."""
    import ctypes

    W = len(src_ptrs)
    Kd = full.shape[1]
    if side == 1:
        M, N = full.shape[0], other.shape[0]
    else:
        M, N = other.shape[0], full.shape[0]
    other = _row_major_2d(other)
    assert other.stride(0) == Kd and full.is_contiguous()
    if out is None:
        out = torch.empty(M, N, dtype=bf16, device=full.device)
    arr = (ctypes.c_void_p * W)(*src_ptrs)
    st = lib.status_tensor(full.device)
    name = "ob_gemm_bf16_ag"
    if _PAIR_AG and rows_per_rank % 256 == 0 and copy_ctas % 2 == 0 and _use_pair(M, N, Kd):
        name = "ob_gemm_bf16_pair_ag"
    _call(name, other.data_ptr(), full.data_ptr(), ctypes.cast(arr, ctypes.c_void_p), out.data_ptr(),
          lib.ptr(residual), M, N, Kd, out.stride(0), residual.stride(0) if residual is not None else 0, 0, side, W,
          rank, rows_per_rank, flags.data_ptr(), int(target) & 0xFFFFFFFF, copy_ctas, st.data_ptr(), lib.stream_ptr())
    return out


def gemm_grouped(a, b, group_offsets, *, b_mn: bool = False, out=None, out_dtype=bf16, pair: bool = False):
    """Ragged-row grouped GEMM.  a: [R,K] rows grouped by ``group_offsets`` (int32 [G+1],
    multiples of 128, R % 128 == 0); b: [G,N,K] (or [G,K,N] when b_mn).  ``pair``: run on CTA pairs
    (256 x 256 tiles); the caller guarantees that every group offset and R are multiples of 256."""
    a = _row_major_2d(a)
    G = b.shape[0]
    R, K = a.shape
    N = b.shape[2] if b_mn else b.shape[1]
    b2 = b.reshape(-1, b.shape[-1])
    lib.check_index("gemm_grouped group_offsets", group_offsets, R + 1)
    if out is None:
        out = torch.empty(R, N, dtype=out_dtype, device=a.device)
    mode = 0 if out.dtype == bf16 else 1
    st = lib.status_tensor(a.device)
    pair = pair and R % 256 == 0
    _call("ob_gemm_bf16_pair_grouped" if pair else "ob_gemm_bf16_grouped", a.data_ptr(), b2.data_ptr(), out.data_ptr(),
          group_offsets.data_ptr(), G, R, N, K, a.stride(0), out.stride(0), int(b_mn), mode,
          st.data_ptr(), lib.stream_ptr())
    return out


def gemm_grouped_wgrad(dy, x, group_offsets, out, accumulate: bool = True, pair: bool = False):
    """out[g] (+)= dy[rows of g]^T x[rows of g]; dy [R,N], x [R,K], out fp32 [G,N,K].  ``pair`` as in
    ``gemm_grouped``."""
    dy = _row_major_2d(dy)
    x = _row_major_2d(x)
    G, N, K = out.shape
    lib.check_index("gemm_grouped_wgrad group_offsets", group_offsets, dy.shape[0] + 1)
    mode = (2 if accumulate else 1) if out.dtype == torch.float32 else 0
    st = lib.status_tensor(dy.device)
    _call("ob_gemm_bf16_pair_grouped_wgrad" if pair else "ob_gemm_bf16_grouped_wgrad", dy.data_ptr(), x.data_ptr(), out.data_ptr(),
          group_offsets.data_ptr(), G, dy.shape[0], N, K, dy.stride(0), x.stride(0), mode,
          st.data_ptr(), lib.stream_ptr())
    return out


def rmsnorm_fwd(x, w, eps, one_plus=False, want_rstd=True):
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = torch.empty_like(x2)
    rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device) if want_rstd else None
    _call("ob_rmsnorm_fwd", x2.data_ptr(), w.data_ptr(), y.data_ptr(), lib.ptr(rstd), x2.shape[0],
          x2.shape[1], float(eps), int(one_plus), lib.stream_ptr())
    return y.view(x.shape), rstd


def rmsnorm_bwd(dy, x, w, rstd, eps, dw_out, one_plus=False):
    x2 = x.reshape(-1, x.shape[-1])
    dy2 = dy.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    if not dy2.is_contiguous():
        dy2 = dy2.contiguous()
    dx = torch.empty_like(x2)
    _call("ob_rmsnorm_bwd", dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), lib.ptr(rstd),
          dx.data_ptr(), lib.ptr(dw_out), x2.shape[0], x2.shape[1], float(eps), int(one_plus),
          lib.stream_ptr())
    return dx.view(x.shape)


def swiglu_fwd(gu):
    g2 = gu.reshape(-1, gu.shape[-1])
    F = g2.shape[1] // 2
    act = torch.empty(g2.shape[0], F, dtype=gu.dtype, device=gu.device)
    _call("ob_swiglu_fwd", g2.data_ptr(), act.data_ptr(), g2.shape[0], F, lib.stream_ptr())
    return act.view(*gu.shape[:-1], F)


def swiglu_bwd(gu, dact, with_act: bool = False, inplace: bool = False):
    """Gradient of silu(gate) * up; ``with_act`` also returns the activation itself, recomputed in
    the same pass (for a caller that did not keep it); ``inplace`` writes the gradient over
    ``gu`` (contiguous), for a caller that is the last reader of it."""
    g2 = gu.reshape(-1, gu.shape[-1])
    F = g2.shape[1] // 2
    d2 = dact.reshape(-1, F)
    if not d2.is_contiguous():
        d2 = d2.contiguous()
    if inplace and not g2.is_contiguous():
        raise ValueError("swiglu_bwd(inplace=True) needs a contiguous [gate | up] tensor")
    dgu = g2 if inplace else torch.empty_like(g2)
    act = torch.empty(g2.shape[0], F, dtype=gu.dtype, device=gu.device) if with_act else None
    _call("ob_swiglu_bwd", g2.data_ptr(), d2.data_ptr(), dgu.data_ptr(), lib.ptr(act), g2.shape[0], F,
          lib.stream_ptr())
    return (dgu.view(gu.shape), act) if with_act else dgu.view(gu.shape)


def qknorm_rope_fwd(qkv, qw, kw, cos, sin, H, G, K, rot, eps, one_plus=False, q_stride_heads=1):
    M = qkv.shape[0]
    q = torch.empty(M, H, K, dtype=qkv.dtype, device=qkv.device)
    k = torch.empty(M, G, K, dtype=qkv.dtype, device=qkv.device)
    _call("ob_qknorm_rope_fwd", qkv.data_ptr(), lib.ptr(qw), lib.ptr(kw), cos.data_ptr(),
          sin.data_ptr(), q.data_ptr(), k.data_ptr(), M, H, G, K, rot, float(eps), int(one_plus),
          q_stride_heads, lib.stream_ptr())
    return q, k


def qknorm_rope_bwd(qkv, qw, kw, cos, sin, dq, dk, dqkv, dqw, dkw, H, G, K, rot, eps,
                    one_plus=False, q_stride_heads=1):
    M = qkv.shape[0]
    _call("ob_qknorm_rope_bwd", qkv.data_ptr(), lib.ptr(qw), lib.ptr(kw), cos.data_ptr(),
          sin.data_ptr(), dq.data_ptr(), dk.data_ptr(), dqkv.data_ptr(), lib.ptr(dqw),
          lib.ptr(dkw), M, H, G, K, rot, float(eps), int(one_plus), q_stride_heads,
          lib.stream_ptr())


def attn_fwd(q, k, v, cu_seqlens, max_seqlen, scale, causal, want_lse=True):
    """q [N,H,K]; k,v [N,G,K] (row-strided views allowed).  Returns out [N,H,K], lse [H,N]."""
    N, H, K = q.shape
    G = k.shape[1]
    for t in (q, k, v):
        if t.stride(2) != 1 or t.stride(1) != K:
            raise ValueError("attention operands need contiguous heads")
    out = torch.empty(N, H, K, dtype=q.dtype, device=q.device)
    lse = torch.empty(H, N, dtype=torch.float32, device=q.device) if want_lse else None
    st = lib.status_tensor(q.device)
    _call("ob_attn_fwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lib.ptr(lse),
          cu_seqlens.data_ptr(), cu_seqlens.numel() - 1, int(max_seqlen), N, H, G, K, q.stride(0),
          k.stride(0), v.stride(0), out.stride(0), float(scale), int(causal), st.data_ptr(),
          lib.stream_ptr())
    return out, lse


_attn_scratch: dict = {}


def attn_bwd(q, k, v, o, lse, do, cu_seqlens, max_seqlen, scale, causal, dk_out=None, dv_out=None):
    """Gradients of ``attn_fwd`` (head_dim 128).  Returns dq [N,H,K], dk, dv [N,G,K].
    ``dk_out`` / ``dv_out`` may be row-strided views (e.g. slices of a fused dqkv buffer).
    The fp32 dq accumulation buffer and the delta vector are cached per shape and reused."""
    N, H, Kd = q.shape
    G = k.shape[1]
    dq = torch.empty(N, H, Kd, dtype=q.dtype, device=q.device)
    dk = dk_out if dk_out is not None else torch.empty(N, G, Kd, dtype=q.dtype, device=q.device)
    dv = dv_out if dv_out is not None else torch.empty(N, G, Kd, dtype=q.dtype, device=q.device)
    key = (q.device.index, N, H, Kd)
    scratch = _attn_scratch.get(key)
    if scratch is None:
        _attn_scratch.clear()
        scratch = (lib.scratch("attn_bwd dq_acc", N * H * Kd, torch.float32, q.device),
                   lib.scratch("attn_bwd delta", H * N, torch.float32, q.device))
        _attn_scratch[key] = scratch
    dq_acc, delta = scratch
    st = lib.status_tensor(q.device)
    _call("ob_attn_bwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(),
          lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(),
          dv.data_ptr(), cu_seqlens.data_ptr(), cu_seqlens.numel() - 1, int(max_seqlen), N, H, G, Kd,
          q.stride(0), k.stride(0), v.stride(0), o.stride(0), do.stride(0), dk.stride(0), dv.stride(0),
          float(scale), int(causal), st.data_ptr(), lib.stream_ptr())
    return dq, dk, dv


def ce_fwd_bwd(logits, targets, mask, grad_scale, loss_sum, write_grad=True, lse_out=None):
    R, V = logits.shape
    _call("ob_ce_fwd_bwd", logits.data_ptr(), logits.stride(0), R, V, targets.data_ptr(),
          lib.ptr(mask), lib.ptr(grad_scale), loss_sum.data_ptr(), lib.ptr(lse_out),
          int(write_grad), lib.stream_ptr())


def sigmoid_gate_fwd(o, gate):
    """o [M,H,Kd] dense, gate [M,H,Kd] (any row / head stride, unit inner stride): o * sigmoid(gate)."""
    M, H, Kd = o.shape
    out = torch.empty_like(o)
    _call("ob_sigmoid_gate_fwd", o.data_ptr(), gate.data_ptr(), out.data_ptr(), M, H, Kd, gate.stride(0), gate.stride(1),
          lib.stream_ptr())
    return out


def sigmoid_gate_bwd(o, gate, dout):
    M, H, Kd = o.shape
    d_o, d_gate = torch.empty_like(o), torch.empty_like(o)
    _call("ob_sigmoid_gate_bwd", o.data_ptr(), gate.data_ptr(), dout.data_ptr(), d_o.data_ptr(), d_gate.data_ptr(), M, H,
          Kd, gate.stride(0), gate.stride(1), lib.stream_ptr())
    return d_o, d_gate


def ce_finish(stats, tgt_logit, mask, loss_sum, lse_out):
    """Row log-sum-exp and masked loss from the statistics the logits GEMM wrote (``gemm(..., ce=)``)."""
    R, n_tiles = stats.shape[0], stats.shape[1]
    _call("ob_ce_finish", stats.data_ptr(), n_tiles, tgt_logit.data_ptr(), lib.ptr(mask), loss_sum.data_ptr(),
          lse_out.data_ptr(), R, lib.stream_ptr())


def embedding_fwd(ids, table):
    ids32 = ids.reshape(-1).to(torch.int32)
    lib.check_index("embedding_fwd ids", ids32, table.shape[0])
    out = torch.empty(ids32.numel(), table.shape[1], dtype=table.dtype, device=table.device)
    _call("ob_embedding_fwd", ids32.data_ptr(), table.data_ptr(), out.data_ptr(), ids32.numel(),
          table.shape[1], lib.stream_ptr())
    return out.view(*ids.shape, table.shape[1])


def embedding_bwd(ids, dy, dtable_f32, row_lo=0, row_hi=None):
    ids32 = ids.reshape(-1).to(torch.int32)
    d2 = dy.reshape(-1, dy.shape[-1])
    if not d2.is_contiguous():
        d2 = d2.contiguous()
    hi = dtable_f32.shape[0] + row_lo if row_hi is None else row_hi
    lib.check_index("embedding_bwd ids", ids32, 2 ** 31 - 1)      # rows outside [row_lo, hi) are skipped, negatives are not expected
    _call("ob_embedding_bwd", ids32.data_ptr(), d2.data_ptr(), dtable_f32.data_ptr(),
          ids32.numel(), d2.shape[1], row_lo, hi, lib.stream_ptr())


def embedding_bwd_peer(ids, dy, peer_ptrs, rows_per_rank: int):
    """Embedding gradient rows added into the owners' fp32 shards over NVLink (``peer_ptrs[r]`` holds
    table rows [r*rows_per_rank, (r+1)*rows_per_rank))."""
    import ctypes

    ids32 = ids.reshape(-1).to(torch.int32)
    d2 = dy.reshape(-1, dy.shape[-1])
    if not d2.is_contiguous():
        d2 = d2.contiguous()
    lib.check_index("embedding_bwd_peer ids", ids32, rows_per_rank * len(peer_ptrs))
    arr = (ctypes.c_void_p * len(peer_ptrs))(*peer_ptrs)
    _call("ob_embedding_bwd_peer", ids32.data_ptr(), d2.data_ptr(), ctypes.cast(arr, ctypes.c_void_p), len(peer_ptrs),
          int(rows_per_rank), ids32.numel(), d2.shape[1], lib.stream_ptr())


def sumsq(g, out):
    _call("ob_sumsq", g.data_ptr(), g.numel(), out.data_ptr(), lib.stream_ptr())


def adamw(p, m, v, g, p16, *, lr, b1, b2, eps, wd, step, grad_mul=1.0, norm_sq=None,
          max_norm=0.0, zero_grad=True):
    bc1 = 1.0 - b1 ** step
    bc2 = 1.0 - b2 ** step
    _call("ob_adamw", p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), lib.ptr(p16),
          p.numel(), float(lr), float(b1), float(b2), float(eps), float(wd), float(bc1),
          float(bc2), float(grad_mul), lib.ptr(norm_sq), float(max_norm), int(zero_grad),
          lib.stream_ptr())


def cast_f32_bf16(src, dst):
    _call("ob_cast_f32_bf16", src.data_ptr(), dst.data_ptr(), src.numel(), lib.stream_ptr())


def transpose(src):
    R, C = src.shape
    dst = torch.empty(C, R, dtype=src.dtype, device=src.device)
    _call("ob_transpose_bf16", src.data_ptr(), dst.data_ptr(), R, C, src.stride(0), dst.stride(0),
          lib.stream_ptr())
    return dst


def l2_flush(buf):
    _call("ob_l2_flush", buf.data_ptr(), buf.numel() * buf.element_size(), lib.stream_ptr())


def decode_append(qkv, qw, kw, positions, seq_of_token, slot_of_token, block_table, page_size, k_pages, v_pages,
                  H, G, HD, rot, theta, eps, one_plus=False):
    """Per-head RMSNorm + RoPE of the new tokens' q and k; k/v go to their page slots.  Returns q."""
    n = qkv.shape[0]
    q = torch.empty(n, H, HD, dtype=qkv.dtype, device=qkv.device)
    _call("ob_decode_append", qkv.data_ptr(), lib.ptr(qw), lib.ptr(kw), positions.data_ptr(),
          seq_of_token.data_ptr(), slot_of_token.data_ptr(), block_table.data_ptr(), block_table.shape[1],
          page_size, q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), n, H, G, HD, rot, float(theta),
          float(eps), int(one_plus), lib.stream_ptr())
    return q


_decode_scratch: dict = {}


def decode_attn(q, k_pages, v_pages, block_table, seq_lens, page_size, scale, splits=None):
    """q [B,H,HD] attends over each sequence's pages; returns [B,H,HD]."""
    B, H, HD = q.shape
    G = k_pages.shape[2]
    if splits is None:
        # the per-key work is latency bound, so fill every SM with ~16 small CTAs, but keep at
        # least 128 keys of cache capacity per split
        cap = block_table.shape[1] * page_size
        splits = max(1, min(32, -(-(148 * 16) // max(B * G, 1)), cap // 128))
    key = (q.device.index, B, H, HD, splits)
    sc = _decode_scratch.get(key)
    if sc is None:
        sc = (torch.empty(B * H * splits * HD, dtype=torch.float32, device=q.device),
              torch.empty(B * H * splits * 2, dtype=torch.float32, device=q.device))
        _decode_scratch[key] = sc
    out = torch.empty_like(q)
    _call("ob_decode_attn", q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
          seq_lens.data_ptr(), B, H, G, HD, block_table.shape[1], page_size, splits, float(scale),
          sc[0].data_ptr(), sc[1].data_ptr(), out.data_ptr(), lib.stream_ptr())
    return out


def causal_conv1d_fwd(x_BTC, w_CK):
    B, T, C = x_BTC.shape
    y = torch.empty_like(x_BTC)
    _call("ob_conv1d_silu_fwd", x_BTC.data_ptr(), w_CK.data_ptr(), y.data_ptr(), B, T, C, w_CK.shape[1], lib.stream_ptr())
    return y


def causal_conv1d_bwd(x_BTC, w_CK, dy, dw_f32):
    B, T, C = x_BTC.shape
    dx = torch.empty_like(x_BTC)
    _call("ob_conv1d_silu_bwd", x_BTC.data_ptr(), w_CK.data_ptr(), dy.data_ptr(), dx.data_ptr(), lib.ptr(dw_f32), B, T, C,
          w_CK.shape[1], lib.stream_ptr())
    return dx


def gdn_fwd(q, k, v, g, beta, s0=None, save=True, want_final=False):
    """Chunked gated delta rule, fp32.  q,k [B,T,Hk,128]; v [B,T,H,U]; g,beta [B,T,H]; T % 64 == 0."""
    B, T, Hk, A = q.shape
    H, U = v.shape[2], v.shape[3]
    o = torch.empty_like(v)
    n_out = torch.empty_like(v) if save else None
    states = torch.empty(B, H, T // 64, A, U, dtype=torch.float32, device=v.device) if save else None
    s_final = torch.empty(B, H, A, U, dtype=torch.float32, device=v.device) if want_final else None
    _call("ob_gdn_fwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), lib.ptr(s0),
          o.data_ptr(), lib.ptr(n_out), lib.ptr(states), lib.ptr(s_final), B, T, H, Hk, A, U, lib.stream_ptr())
    return o, n_out, states, s_final


def gdn_bwd(q, k, v, g, beta, n_out, states, d_o, d_sfinal=None, want_ds0=False):
    B, T, Hk, A = q.shape
    H, U = v.shape[2], v.shape[3]
    dq, dk = torch.zeros_like(q), torch.zeros_like(k)
    dv = torch.empty_like(v)
    dg, dbeta = torch.zeros_like(g), torch.zeros_like(beta)
    ds0 = torch.empty(B, H, A, U, dtype=torch.float32, device=v.device) if want_ds0 else None
    _call("ob_gdn_bwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), n_out.data_ptr(),
          states.data_ptr(), d_o.data_ptr(), lib.ptr(d_sfinal), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
          dg.data_ptr(), dbeta.data_ptr(), lib.ptr(ds0), B, T, H, Hk, A, U, lib.stream_ptr())
    return dq, dk, dv, dg, dbeta, ds0


def gated_rmsnorm_fwd(x, z, w, eps):
    M, D = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    _call("ob_gated_rmsnorm_fwd", x.data_ptr(), z.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), M, D,
          float(eps), lib.stream_ptr())
    return y, rstd


def gated_rmsnorm_bwd(dy, x, z, w, rstd, eps, dw_f32):
    M, D = x.shape
    dx, dz = torch.empty_like(x), torch.empty_like(z)
    _call("ob_gated_rmsnorm_bwd", dy.data_ptr(), x.data_ptr(), z.data_ptr(), w.data_ptr(), lib.ptr(rstd), dx.data_ptr(),
          dz.data_ptr(), dw_f32.data_ptr(), M, D, float(eps), lib.stream_ptr())
    return dx, dz


def layernorm_fwd(x, w, b, eps):
    M, D = x.shape
    y = torch.empty_like(x)
    mean = torch.empty(M, dtype=torch.float32, device=x.device)
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    _call("ob_layernorm_fwd", x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
          M, D, float(eps), lib.stream_ptr())
    return y, mean, rstd


def layernorm_bwd(dy, x, w, mean, rstd, dw_f32, db_f32):
    M, D = x.shape
    dx = torch.empty_like(x)
    _call("ob_layernorm_bwd", dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
          dw_f32.data_ptr(), db_f32.data_ptr(), M, D, lib.stream_ptr())
    return dx


def router_topk(logits, k, renorm, counts=None):
    """logits [M,E] bf16 -> probs [M,E] fp32, weights [M,k] fp32, idx [M,k] int32; counts [E] int32 += picks."""
    M, E = logits.shape
    probs = torch.empty(M, E, dtype=torch.float32, device=logits.device)
    w = torch.empty(M, k, dtype=torch.float32, device=logits.device)
    idx = torch.empty(M, k, dtype=torch.int32, device=logits.device)
    _call("ob_router_topk", logits.data_ptr(), probs.data_ptr(), w.data_ptr(), idx.data_ptr(), lib.ptr(counts), M, E, k,
          int(renorm), lib.stream_ptr())
    return probs, w, idx


def router_topk_bwd(probs, w, idx, dw, dprobs, renorm):
    M, E = probs.shape
    dlogits = torch.empty(M, E, dtype=bf16, device=probs.device)
    _call("ob_router_topk_bwd", probs.data_ptr(), w.data_ptr(), idx.data_ptr(), dw.data_ptr(), lib.ptr(dprobs),
          dlogits.data_ptr(), M, E, idx.shape[1], int(renorm), lib.stream_ptr())
    return dlogits


def moe_plan(idx32, E, pad=128, counts=None):
    """idx [M,k] int32 -> offsets [E+1] int32 (segments padded to ``pad``), dest [M*k] int32.
    ``counts`` [E] int32 may carry the histogram already (from the router)."""
    have = counts is not None
    if not have:
        counts = torch.empty(E, dtype=torch.int32, device=idx32.device)
    Pn = idx32.numel()
    offsets = torch.empty(E + 1, dtype=torch.int32, device=idx32.device)
    cursor = torch.empty(E, dtype=torch.int32, device=idx32.device)
    dest = torch.empty(Pn, dtype=torch.int32, device=idx32.device)
    _call("ob_moe_plan", idx32.data_ptr(), counts.data_ptr(), offsets.data_ptr(), cursor.data_ptr(), dest.data_ptr(), Pn,
          E, pad, int(not have), lib.stream_ptr())
    return offsets, dest


def gather_rows(src, idx32):
    out = torch.empty(idx32.numel(), src.shape[1], dtype=src.dtype, device=src.device)
    _call("ob_gather_rows", src.data_ptr(), idx32.data_ptr(), out.data_ptr(), idx32.numel(), src.shape[1], lib.stream_ptr())
    return out


def scatter_rows_(dst, idx32, src, replace: bool):
    _call("ob_scatter_rows", dst.data_ptr(), idx32.data_ptr(), src.data_ptr(), idx32.numel(), dst.shape[1], int(replace),
          lib.stream_ptr())
    return dst


def gather4_fwd(table, idx32_N4, w_N4):
    n = idx32_N4.shape[0]
    lib.check_index("gather4 idx", idx32_N4, table.shape[0])
    out = torch.empty(n, table.shape[1], dtype=table.dtype, device=table.device)
    _call("ob_gather4_fwd", table.data_ptr(), idx32_N4.data_ptr(), w_N4.data_ptr(), out.data_ptr(), n, table.shape[1],
          lib.stream_ptr())
    return out


def gather4_bwd(dout, idx32_N4, w_N4, dtable_f32):
    lib.check_index("gather4 idx", idx32_N4, dtable_f32.shape[0])
    _call("ob_gather4_bwd", dout.data_ptr(), idx32_N4.data_ptr(), w_N4.data_ptr(), dtable_f32.data_ptr(), idx32_N4.shape[0],
          dout.shape[1], lib.stream_ptr())


def gelu_tanh_fwd(x):
    y = torch.empty_like(x)
    _call("ob_gelu_tanh_fwd", x.data_ptr(), y.data_ptr(), x.numel(), lib.stream_ptr())
    return y


def gelu_tanh_bwd(x, dy):
    dx = torch.empty_like(x)
    _call("ob_gelu_tanh_bwd", x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel(), lib.stream_ptr())
    return dx


def ce_vp_stats(logits, targets32, v0):
    R, V = logits.shape
    mx, sm, tg = (torch.empty(R, dtype=torch.float32, device=logits.device) for _ in range(3))
    _call("ob_ce_vp_stats", logits.data_ptr(), R, V, logits.stride(0), int(v0), targets32.data_ptr(), mx.data_ptr(),
          sm.data_ptr(), tg.data_ptr(), lib.stream_ptr())
    return mx, sm, tg


def ce_vp_grad_(logits, targets32, v0, lse, mask, grad_scale):
    R, V = logits.shape
    _call("ob_ce_vp_grad", logits.data_ptr(), R, V, logits.stride(0), int(v0), targets32.data_ptr(), lse.data_ptr(),
          lib.ptr(mask), lib.ptr(grad_scale), lib.stream_ptr())
    return logits
