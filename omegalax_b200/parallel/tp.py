"""Tensor parallelism with sequence-parallel activations (Megatron style).

Between blocks every tp rank holds M/tp rows of the activations.  A column-parallel
projection (QKV, gate/up) first all-gathers the rows, a row-parallel projection (o, down)
ends in a reduce-scatter over rows:

    column:  y_local_cols[M, N/tp] = all_gather_rows(x[M/tp, D]) @ W_r^T
    row:     y[M/tp, D]            = reduce_scatter_rows(x_local_cols[M, F/tp] @ W_r^T) + residual

Transports.  "p2p" (CUDA, bf16): the gather is the pull kernel over NVLink peer pointers into a
local staging buffer that the tcgen05 GEMM then reads; the row-parallel GEMM uses the
peer-reduce epilogue, i.e. every output tile is added (fp32) directly into the owning rank's
rows over NVLink -- GEMM and reduce-scatter are one kernel.  "dist": torch.distributed
collectives (NCCL baseline, gloo on CPU ranks).  The reference shards heads / mlp over a "tp"
mesh axis and lets the compiler insert all-reduces (omegalax/models/shard_config.py:12-24); it
has no sequence parallelism.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import functional as Fn
from ..ops import kernels as K

_ACTIVE: "TPContext | None" = None


def current() -> "TPContext | None":
    return _ACTIVE


def set_current(ctx: "TPContext | None") -> None:
    global _ACTIVE
    _ACTIVE = ctx


class TPContext:
    def __init__(self, group, transport: str = "auto"):
        self.group = group
        self.size = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        if transport == "auto":
            transport = "p2p" if (torch.cuda.is_available() and self.size > 1
                                  and dist.get_backend(group) == "nccl") else "dist"
        self.transport = transport
        self._gather_buf = None
        self._rs_buf = None
        self._barrier = None
        self._ag_bufs = [None, None]   # alternating staging buffers of the fused gather + GEMM
        self._ag_calls = 0
        self._ag_flags = None
        self._ag_count = 0             # value of the chunk counters after the calls issued so far

    # ---- peer-memory resources (allocated on first use, sized by the largest request)
    def _symm(self):
        from . import symm

        return symm

    def gather_buffer(self, rows_local: int, cols: int, dtype):
        n = rows_local * cols * 2
        if self._gather_buf is None or self._gather_buf.nbytes < n:
            self._gather_buf = self._symm().SymmetricBuffer(n, self.group)
            if self._barrier is None:
                self._barrier = self._symm().DeviceBarrier(self.group)
        return self._gather_buf

    def ag_stage(self, nbytes: int):
        """Staging buffer for this call of the fused gather + GEMM, the per-chunk counters and the
        value they reach when this call's chunks are complete.  Two buffers alternate: a buffer is
        rewritten two calls later, and the barrier of the call in between proves that every peer
        has finished reading it."""
        i = self._ag_calls & 1
        if self._ag_bufs[i] is None or self._ag_bufs[i].nbytes < nbytes:
            self._ag_bufs[i] = self._symm().SymmetricBuffer(nbytes, self.group)
        if self._barrier is None:
            self._barrier = self._symm().DeviceBarrier(self.group)
        if self._ag_flags is None:
            self._ag_flags = torch.zeros(self.size, dtype=torch.int32, device="cuda")
        self._ag_calls += 1
        return self._ag_bufs[i], self._ag_flags

    def rs_buffer(self, rows_local: int, cols: int):
        n = rows_local * cols * 2
        if self._rs_buf is None or self._rs_buf.nbytes < n:
            self._rs_buf = self._symm().SymmetricBuffer(n, self.group)
            if self._barrier is None:
                self._barrier = self._symm().DeviceBarrier(self.group)
        return self._rs_buf


# ----------------------------------------------------------------------------- collectives
def _ag_rows(x, tp: TPContext):
    m, D = x.shape
    out = torch.empty(m * tp.size, D, dtype=x.dtype, device=x.device)
    if tp.transport == "p2p" and x.dtype == torch.bfloat16:
        symm = tp._symm()
        buf = tp.gather_buffer(m, D, x.dtype)
        buf.view(x.dtype, m * D).copy_(x.reshape(-1))
        tp._barrier()
        tab = symm.make_copy_segments([(r, 0, r * m * D * 2, m * D * 2) for r in range(tp.size)], x.device)
        symm.allgather_pull(buf, out, tab)
        tp._barrier()  # peers have finished reading before the staging buffer is reused
    else:
        dist.all_gather_into_tensor(out, x.contiguous(), group=tp.group)
    return out


def _rs_rows(y, tp: TPContext):
    M, D = y.shape
    m = M // tp.size
    out = torch.empty(m, D, dtype=y.dtype, device=y.device)
    dist.reduce_scatter_tensor(out, y.contiguous(), op=dist.ReduceOp.SUM, group=tp.group)
    return out


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _ag_rows(x, tp)

    @staticmethod
    def backward(ctx, g):
        return _rs_rows(g, ctx.tp), None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, tp):
        ctx.tp = tp
        return _rs_rows(y, tp)

    @staticmethod
    def backward(ctx, g):
        return _ag_rows(g.contiguous(), ctx.tp), None


class replicated_rows:
    """Context manager for inference with a KV cache: every tensor-parallel rank carries all rows
    (a decode step has too few rows to split), so the gathers become no-ops and a row-parallel
    projection ends in an all-reduce instead of a reduce-scatter.  No autograd support."""

    def __init__(self, tp: "TPContext | None"):
        self.tp = tp

    def __enter__(self):
        if self.tp is not None:
            self.prev, self.tp.replicated = getattr(self.tp, "replicated", False), True
        return self

    def __exit__(self, *a):
        if self.tp is not None:
            self.tp.replicated = self.prev


def _replicated(tp) -> bool:
    return tp is not None and getattr(tp, "replicated", False)


def all_gather_rows(x, tp: TPContext | None):
    if tp is None or tp.size == 1 or _replicated(tp):
        return x
    return _AllGatherRows.apply(x, tp)


def reduce_scatter_rows(y, tp: TPContext | None):
    if tp is None or tp.size == 1:
        return y
    return _ReduceScatterRows.apply(y, tp)


# ----------------------------------------------------------------------------- fused row-parallel
def _rs_mode(tp: "TPContext") -> str:
    """How a GEMM's result rows reach their owners.  "atomic": the epilogue adds every tile into the
    owner's rows with vector bf16 reductions (one pass, best for two ranks); "staged": the epilogue
    stores the tile into the sender's slab of the owner's staging buffer with plain 16-byte stores
    and the owner sums the slabs (wider groups, where the reduction rate of the atomics, not the
    link, was the bound: 0.09 of the NVLink roofline at eight ranks)."""
    forced = os.environ.get("OMEGALAX_B200_TP_RS")
    if forced in ("atomic", "staged"):
        return forced
    return "atomic" if tp.size <= 2 else "staged"


def _gemm_reduce_scatter(x, w, tp: "TPContext", *, b_mn: bool, residual=None):
    """rows [r*m, (r+1)*m) of x @ op(w), summed over the tensor-parallel ranks, land on rank r
    (+ residual): GEMM and reduce-scatter over NVLink peer memory, no library collective."""
    M = x.shape[0]
    N = w.shape[1] if b_mn else w.shape[0]
    m = M // tp.size
    if _rs_mode(tp) == "atomic":
        buf = tp.rs_buffer(m, N)
        acc = buf.view(torch.bfloat16, m * N)
        acc.zero_()
        tp._barrier()                                   # every owner has cleared its rows
        K.gemm_peer_reduce(x, w, buf.peer_ptr_list(0), m, N, b_mn=b_mn, bf16_out=True)
        tp._barrier()                                   # all contributions have landed
        return acc.view(m, N) + residual if residual is not None else acc.view(m, N).clone()
    buf = tp.rs_buffer(m * tp.size, N)                  # one [m, N] slab per sender
    tp._barrier()                                       # every owner has summed the previous call's slabs
    K.gemm_peer_reduce(x, w, buf.peer_ptr_list(0), m, N, b_mn=b_mn, slot=tp.rank)
    tp._barrier()                                       # all slabs have landed
    out = torch.empty(m, N, dtype=torch.bfloat16, device=x.device)
    res = residual.contiguous() if residual is not None else None
    return K.slab_sum(buf.view(torch.bfloat16, tp.size * m * N), tp.size, out, res)


class _RowParallelLinearFn(torch.autograd.Function):
    """y[M/tp, N] = reduce_scatter_rows(x[M, K/tp] @ w[N, K/tp]^T) (+ residual), with the
    reduce-scatter performed by the GEMM epilogue over NVLink peer memory."""

    @staticmethod
    def forward(ctx, x, w, residual, tp: TPContext):
        y = _gemm_reduce_scatter(x, w, tp, b_mn=False, residual=residual)
        ctx.save_for_backward(x, w)
        ctx.tp, ctx.w_ref, ctx.has_res = tp, w, residual is not None
        return y

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        tp = ctx.tp
        gfull = _ag_rows(g.contiguous(), tp)            # [M, N]
        dx = K.gemm(gfull, w, b_mn=True)
        mg = getattr(ctx.w_ref, "main_grad", None)
        pg = getattr(ctx.w_ref, "peer_grad", None)
        dw = None
        if pg is not None:
            K.gemm_peer_reduce(gfull, x, pg[0], pg[1], pg[2], a_mn=True, b_mn=True)
        elif mg is not None:
            K.gemm(gfull, x, a_mn=True, b_mn=True, out=mg, accumulate=True)
        else:
            dw = K.gemm(gfull, x, a_mn=True, b_mn=True)
        return dx, dw, (g if ctx.has_res else None), None


class _ColumnParallelLinearFn(torch.autograd.Function):
    """y[M, N/tp] = all_gather_rows(x[M/tp, K]) @ w[N/tp, K]^T with the gather running inside the
    GEMM launch (copy CTAs stream the peers' row chunks in while the tiles of the chunks that
    have arrived are computed).  Backward: the input gradient GEMM reduce-scatters in its epilogue."""

    @staticmethod
    def forward(ctx, x, w, tp: TPContext):
        m, Kd = x.shape
        stage, flags = tp.ag_stage(m * Kd * 2)
        stage.view(x.dtype, m * Kd).copy_(x.reshape(-1))
        tp._barrier()                                   # every rank's chunk is in its staging buffer
        full = torch.empty(m * tp.size, Kd, dtype=x.dtype, device=x.device)
        ctas = K.ag_copy_ctas(m * tp.size, w.shape[0], Kd, tp.size * m * Kd * 2.0)
        tp._ag_count += ctas
        y = K.gemm_ag(w, full, stage.peer_ptr_list(0), side=1, rank=tp.rank, rows_per_rank=m, flags=flags,
                      target=tp._ag_count, copy_ctas=ctas)
        ctx.save_for_backward(full, w)
        ctx.tp, ctx.w_ref = tp, w
        return y

    @staticmethod
    def backward(ctx, dy):
        full, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        M, Kd = full.shape
        m = M // tp.size
        dx = _gemm_reduce_scatter(dy, w, tp, b_mn=True)     # dx rows land on their owners
        mg = getattr(ctx.w_ref, "main_grad", None)
        pg = getattr(ctx.w_ref, "peer_grad", None)
        dw = None
        if pg is not None:
            K.gemm_peer_reduce(dy, full, pg[0], pg[1], pg[2], a_mn=True, b_mn=True)
        elif mg is not None:
            K.gemm(dy, full, a_mn=True, b_mn=True, out=mg, accumulate=True)
        else:
            dw = K.gemm(dy, full, a_mn=True, b_mn=True)
        return dx, dw, None


def column_parallel_linear(x_local, w_local, tp: TPContext | None):
    """all-gather rows -> projection with this rank's output columns."""
    if _replicated(tp):
        return Fn.linear(x_local, w_local)
    if tp is not None and tp.size > 1 and tp.transport == "p2p" and Fn.use_kernels(x_local) \
            and w_local.dtype == torch.bfloat16 and x_local.dim() == 2 and x_local.shape[0] % 128 == 0 \
            and x_local.shape[1] % 8 == 0 and w_local.shape[0] % 8 == 0:
        return _ColumnParallelLinearFn.apply(x_local.contiguous(), w_local, tp)
    return Fn.linear(all_gather_rows(x_local, tp), w_local)


def row_parallel_linear(x_cols, w_local, residual_local, tp: TPContext | None):
    """projection over this rank's input columns -> reduce-scatter over rows (+ residual)."""
    if tp is None or tp.size == 1:
        return Fn.linear(x_cols, w_local, residual=residual_local)
    if _replicated(tp):   # all rows on every rank: sum the partial products over tp
        y = Fn.linear(x_cols, w_local).contiguous()
        dist.all_reduce(y, group=tp.group)
        return y if residual_local is None else y + residual_local
    # GEMM and reduce-scatter over peer memory at every group size: vector atomics in the epilogue for
    # two ranks, per-sender slabs summed by the owner for wider groups (see _rs_mode).
    if tp.transport == "p2p" and Fn.use_kernels(x_cols) and w_local.dtype == torch.bfloat16 \
            and w_local.shape[0] % 8 == 0 and os.environ.get("OMEGALAX_B200_TP_RS") != "nccl":
        return _RowParallelLinearFn.apply(x_cols.contiguous(), w_local, residual_local, tp)
    y = reduce_scatter_rows(Fn.linear(x_cols, w_local), tp)
    return y if residual_local is None else y + residual_local


# ----------------------------------------------------------------------------- weight slicing
def slice_rows(t, tp: int, rank: int):
    n = t.shape[0] // tp
    return t[rank * n:(rank + 1) * n]


def slice_cols(t, tp: int, rank: int):
    n = t.shape[1] // tp
    return t[:, rank * n:(rank + 1) * n]


def qkv_rows_for_rank(H: int, G: int, Kd: int, tp: int, rank: int, q_mult: int = 1) -> torch.Tensor:
    """Row indices of a fused [q | k | v] projection that belong to one tp rank: its query
    heads, its kv heads (keys) and its kv heads (values)."""
    Hl, Gl = H // tp, G // tp
    q = torch.arange(rank * Hl * Kd * q_mult, (rank + 1) * Hl * Kd * q_mult)
    k0 = H * Kd * q_mult
    k = torch.arange(k0 + rank * Gl * Kd, k0 + (rank + 1) * Gl * Kd)
    v0 = k0 + G * Kd
    v = torch.arange(v0 + rank * Gl * Kd, v0 + (rank + 1) * Gl * Kd)
    return torch.cat([q, k, v])


def gate_up_rows_for_rank(F: int, tp: int, rank: int) -> torch.Tensor:
    Fl = F // tp
    return torch.cat([torch.arange(rank * Fl, (rank + 1) * Fl), torch.arange(F + rank * Fl, F + (rank + 1) * Fl)])
