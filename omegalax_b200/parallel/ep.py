"""Expert parallelism: experts are sharded over the data ranks and tokens travel to them.

Rank r owns experts [r*E/W, (r+1)*E/W).  One MoE layer runs as

    plan      every rank stores its per-expert pair counts into all peers' count tables (one small
              kernel and a device barrier, no host-launched collective); every rank then derives
              the same row layout of every receive buffer: per local expert, the senders'
              segments in rank order, each expert padded to a multiple of PAD rows
    dispatch  each (token, slot) row is written straight into the owner's receive buffer at
              its final row -- router permutation and all-to-all in one kernel (peer stores)
    experts   grouped tcgen05 GEMMs + SwiGLU on the local receive buffer
    combine   every token pulls its k expert outputs from the owners (peer loads) and forms the
              weighted sum in fp32 -- all-to-all and weighted un-permute in one kernel

The backward uses the same two kernels with the roles swapped (a scaled push for the combine,
a pull for the dispatch, plus a pull that returns the per-pair dot products for the routing
weight gradient).  Cross-GPU ordering uses the bounded device barrier.  The reference has no
expert parallelism (it evaluates every expert for every token: omegalax/models/qwen3/model.py:92-104).

``ExpertParallelA2A`` at the end of this file is the same contract on library collectives
(``all_to_all_single``): the baseline for the kernels above, the fallback without peer memory and
the form that runs on CPU ranks; it is also the transport when the experts are cut over shard
group x tensor-parallel group.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import lib
from ..ops import moe as moe_ops
from . import symm

PAD = moe_ops.PAD    # expert segments are padded to this many rows (256: grouped GEMMs on CTA pairs)


def _register():
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    lib.register("ob_ep_push", [P, I, P, P, P, P, P, L, I, P])
    lib.register("ob_ep_pull", [P, I, P, P, P, P, P, P, L, I, I, P])
    lib.register("ob_ep_publish_counts", [P, I, I, P, I, P])


_register()


class Plan:
    """Row assignment of one MoE layer call (device tensors, no host sync)."""
    __slots__ = ("dst_rank", "dst_row", "src_tok", "offsets_local", "M", "k", "overflow")


def build_plan(idx, E: int, W: int, rank: int, group, capacity: int) -> Plan:
    """idx [M,k] global expert ids -> destination (rank, row) of every pair and the local
    group offsets of this rank's receive buffer."""
    M, k = idx.shape
    dev = idx.device
    El = E // W
    flat = idx.reshape(-1)
    counts = torch.bincount(flat, minlength=E).to(torch.int32)             # my pairs per global expert
    allc = torch.empty(W, E, dtype=torch.int32, device=dev)
    if W > 1:
        dist.all_gather_into_tensor(allc.view(-1), counts, group=group)
    else:
        allc[0] = counts
    allc = allc.to(torch.int64)
    tot = allc.sum(0)                                                      # rows per global expert
    padded = (tot + PAD - 1) // PAD * PAD
    pe = padded.view(W, El)
    base_e = (pe.cumsum(1) - pe).reshape(-1)                               # start of expert inside its owner's buffer
    before_me = allc[:rank].sum(0) if rank > 0 else torch.zeros(E, dtype=torch.int64, device=dev)
    # rank of every pair among my pairs of the same expert (stable sort)
    order = torch.argsort(flat, stable=True)
    starts = counts.to(torch.int64).cumsum(0) - counts.to(torch.int64)
    sorted_e = flat[order]
    r_in_e = torch.arange(flat.numel(), device=dev) - starts[sorted_e]
    row_sorted = base_e[sorted_e] + before_me[sorted_e] + r_in_e
    dst_row = torch.empty_like(row_sorted)
    dst_row[order] = row_sorted
    p = Plan()
    p.dst_rank = (flat // El).to(torch.int32)
    p.dst_row = dst_row.to(torch.int32)
    p.src_tok = torch.arange(M, device=dev, dtype=torch.int32).repeat_interleave(k)
    mine = pe[rank]
    offs = torch.zeros(El + 1, dtype=torch.int64, device=dev)
    offs[1:] = mine.cumsum(0)
    p.offsets_local = offs.to(torch.int32)
    p.M, p.k = M, k
    p.overflow = (pe.sum(1).max() > capacity)                             # checked lazily by the caller
    return p


def build_plan_device(idx, E: int, W: int, rank: int, group, capacity: int, overflow_flag, src_tok, ep=None) -> Plan:
    """Same plan as ``build_plan`` from kernel launches only.  With ``ep`` (an ``ExpertParallel``)
    every rank stores its counts into all peers' count tables and the device barrier that follows
    doubles as the "previous contents consumed" barrier of the dispatch; without it the counts are
    all-gathered by the process group.  Rows of one sender inside an expert segment are assigned by
    an atomic cursor, so their order (not their set) can differ from run to run."""
    M, k = idx.shape
    dev = idx.device
    idx32 = idx.reshape(-1).to(torch.int32)
    lib.check_index("expert ids", idx32, E)
    if ep is not None and W > 1:
        allc = ep.count_table
        mine = ep.my_counts
        lib.call("ob_moe_count", idx32.data_ptr(), mine.data_ptr(), idx32.numel(), E, lib.stream_ptr())
        lib.call("ob_ep_publish_counts", ep.count_buf.ptr_table(), W, rank, mine.data_ptr(), E, lib.stream_ptr())
        ep.barrier()      # counts of every rank have landed; every rank is done with the previous exchange
    else:
        allc = torch.empty(W, E, dtype=torch.int32, device=dev)
        mine = allc[rank]
        lib.call("ob_moe_count", idx32.data_ptr(), mine.data_ptr(), idx32.numel(), E, lib.stream_ptr())
        if W > 1:
            dist.all_gather_into_tensor(allc.view(-1), mine.clone(), group=group)
    p = Plan()
    scratch = torch.empty(2 * E, dtype=torch.int32, device=dev)
    p.offsets_local = torch.empty(E // W + 1, dtype=torch.int32, device=dev)
    p.dst_rank = torch.empty(M * k, dtype=torch.int32, device=dev)
    p.dst_row = torch.empty(M * k, dtype=torch.int32, device=dev)
    lib.call("ob_ep_plan", idx32.data_ptr(), allc.data_ptr(), scratch.data_ptr(), p.offsets_local.data_ptr(),
             p.dst_rank.data_ptr(), p.dst_row.data_ptr(), overflow_flag.data_ptr(), M * k, W, E, rank, PAD, capacity,
             lib.stream_ptr())
    p.src_tok = src_tok
    p.M, p.k = M, k
    p.overflow = None
    return p


class ExpertParallel:
    def __init__(self, group, num_experts: int, hidden: int, max_tokens: int, top_k: int, *,
                 capacity_factor: float = 2.0, dtype=torch.bfloat16, reuse_buffers: bool = False):
        self.group = group
        self.W = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        if num_experts % self.W:
            raise ValueError(f"{num_experts} experts do not divide over {self.W} ranks")
        self.E, self.D, self.El = num_experts, hidden, num_experts // self.W
        cap = int(capacity_factor * max_tokens * top_k) + self.El * (PAD - 1)
        self.capacity = (cap + PAD - 1) // PAD * PAD
        nbytes = self.capacity * hidden * 2
        # receive buffers: token rows in, expert outputs, and their two gradient counterparts
        self.buf_in = symm.SymmetricBuffer(nbytes, group)
        self.buf_out = symm.SymmetricBuffer(nbytes, group)
        self.buf_gout = symm.SymmetricBuffer(nbytes, group)
        self.buf_gin = symm.SymmetricBuffer(nbytes, group)
        self.barrier = symm.DeviceBarrier(group)
        # per-expert pair counts of every rank, written by the peers themselves (no host collective)
        self.count_buf = symm.SymmetricBuffer(max(self.W * self.E * 4, 256), group)
        self.count_table = self.count_buf.view(torch.int32, self.W * self.E).view(self.W, self.E)
        self.my_counts = torch.zeros(self.E, dtype=torch.int32, device="cuda")
        self.dtype = dtype
        self.overflow_flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        self._src_tok = {}
        # With layer-by-layer rematerialisation (every policy but "none": the layer is re-run in its
        # backward, with or without stashed outputs) a layer's exchange buffers are consumed before
        # the next layer touches them, so the expert MLP can read and write them in place.  The
        # buffers start zeroed and only ever hold finite activations afterwards: padding rows may
        # then carry stale values, which is harmless because the gradient of the expert output is
        # always zero on padding rows (so no weight gradient sees them).
        self.reuse_buffers = reuse_buffers
        for b in (self.buf_in, self.buf_out, self.buf_gout, self.buf_gin):
            self.local(b).zero_()
        self.barrier()

    def local(self, buf: symm.SymmetricBuffer) -> torch.Tensor:
        return buf.view(self.dtype, self.capacity * self.D).view(self.capacity, self.D)

    def push(self, buf, src, plan: Plan, scale=None):
        lib.call("ob_ep_push", buf.ptr_table(), self.W, src.data_ptr(), plan.src_tok.data_ptr(),
                 plan.dst_rank.data_ptr(), plan.dst_row.data_ptr(), lib.ptr(scale), plan.M * plan.k, self.D,
                 lib.stream_ptr())

    def pull(self, buf, plan: Plan, weights=None, out=True, grad=None):
        o = torch.empty(plan.M, self.D, dtype=self.dtype, device="cuda") if out else None
        dots = torch.empty(plan.M * plan.k, dtype=torch.float32, device="cuda") if grad is not None else None
        lib.call("ob_ep_pull", buf.ptr_table(), self.W, lib.ptr(o), plan.dst_rank.data_ptr(), plan.dst_row.data_ptr(),
                 lib.ptr(weights), lib.ptr(grad), lib.ptr(dots), plan.M, plan.k, self.D, lib.stream_ptr())
        return o, dots

    def check(self):
        if bool(self.overflow_flag.item()):
            raise RuntimeError("expert-parallel receive buffer overflow: raise capacity_factor")

    def moe_mlp(self, x, weights, idx, w_gate_up_local, w_down_local):
        """x [M,D] local tokens; weights/idx [M,k]; expert weights are this rank's E/W experts."""
        key = tuple(idx.shape)
        st = self._src_tok.get(key)
        if st is None:
            st = torch.arange(idx.shape[0], device=idx.device, dtype=torch.int32).repeat_interleave(idx.shape[1])
            self._src_tok[key] = st
        if not self.reuse_buffers:
            self.local(self.buf_in).zero_()       # padding rows start from zero (before the barrier inside the plan)
        plan = build_plan_device(idx, self.E, self.W, self.rank, self.group, self.capacity, self.overflow_flag, st,
                                 ep=self)
        xp = _Dispatch.apply(x.contiguous(), self, plan)
        out = self.local(self.buf_out) if self.reuse_buffers else None
        yp = moe_ops.expert_mlp_permuted(xp, w_gate_up_local, w_down_local, plan.offsets_local, out)
        return _Combine.apply(yp, weights.contiguous().float(), self, plan)


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ep: ExpertParallel, plan: Plan):
        if ep.W == 1:
            ep.barrier()                      # (with peers the plan's count exchange has already synchronised)
        ep.push(ep.buf_in, x, plan)
        ep.barrier()                          # all rows have landed
        ctx.ep, ctx.plan = ep, plan
        return ep.local(ep.buf_in) if ep.reuse_buffers else ep.local(ep.buf_in).clone()

    @staticmethod
    def backward(ctx, d_xp):
        ep, plan = ctx.ep, ctx.plan
        ep.local(ep.buf_gin).copy_(d_xp)
        ep.barrier()
        dx, _ = ep.pull(ep.buf_gin, plan, weights=None)
        ep.barrier()                          # peers are done reading before the buffer is reused
        return dx, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, yp, weights, ep: ExpertParallel, plan: Plan):
        ctx.in_place = yp.data_ptr() == ep.local(ep.buf_out).data_ptr()
        if not ctx.in_place:
            ep.local(ep.buf_out).copy_(yp)
        ep.barrier()
        y, _ = ep.pull(ep.buf_out, plan, weights=weights.reshape(-1))
        ep.barrier()
        ctx.ep, ctx.plan = ep, plan
        ctx.save_for_backward(weights, yp)
        return y

    @staticmethod
    def backward(ctx, dy):
        ep, plan = ctx.ep, ctx.plan
        weights, yp = ctx.saved_tensors
        dy = dy.contiguous()
        # gradient of the routing weights: <dy[token], expert output row>
        if not ctx.in_place:                  # in place: the recomputation has just rewritten it
            ep.local(ep.buf_out).copy_(yp)
        ep.local(ep.buf_gout).zero_()         # padding rows of the output gradient must be zero
        ep.barrier()
        _, dots = ep.pull(ep.buf_out, plan, weights=None, out=False, grad=dy)
        # gradient of the expert outputs: weight * dy[token], pushed to the owners
        ep.push(ep.buf_gout, dy, plan, scale=weights.reshape(-1))
        ep.barrier()
        # consumed by the expert MLP's backward before any other layer writes this buffer
        return ep.local(ep.buf_gout), dots.view_as(weights), None, None


# ----------------------------------------------------------------------------- library path
class _AllToAllRows(torch.autograd.Function):
    """``dist.all_to_all_single`` over row blocks; the gradient travels the same way back."""

    @staticmethod
    def forward(ctx, rows, send_counts, recv_counts, group):
        ctx.group, ctx.send, ctx.recv = group, send_counts, recv_counts
        out = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        back = g.new_empty((sum(ctx.send),) + tuple(g.shape[1:]))
        dist.all_to_all_single(back, g.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv,
                               group=ctx.group)
        return back, None, None, None


class ExpertParallelA2A:
    """Expert parallelism on library collectives: the same contract as ``ExpertParallel.moe_mlp``
    (rank r owns experts [r*E/W, (r+1)*E/W); every (token, slot) pair is computed by the rank that
    owns its expert), moved with two ``all_to_all_single`` calls per direction instead of the
    peer-memory kernels.  It is the baseline those kernels are measured against, the fallback
    where GPUs cannot map each other's memory, and the form that runs on CPU ranks (gloo) in the
    tests.  One host synchronisation per layer (the split sizes are host integers); no capacity
    limit, nothing is ever dropped."""

    def __init__(self, group, num_experts: int):
        self.group = group
        self.W = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        if num_experts % self.W:
            raise ValueError(f"{num_experts} experts do not divide over {self.W} ranks")
        self.E, self.El = num_experts, num_experts // self.W
        self.max_tokens = 1 << 62

    def check(self):          # same surface as the peer-memory exchange; nothing can overflow here
        return None

    def moe_mlp(self, x, w, idx, gate_up_local, down_local):
        from ..ops import moe as moe_ops

        M, D = x.shape
        k = idx.shape[1]
        pair_e = idx.reshape(-1).long()                               # expert of pair p = token * k + slot
        order = torch.argsort(pair_e, stable=True)                    # pairs grouped by expert, hence by owner
        e_sorted = pair_e[order]
        send = torch.bincount(e_sorted // self.El, minlength=self.W)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        send_l, recv_l = send.tolist(), recv.tolist()
        rows = x.index_select(0, order // k)                          # differentiable gather of the token rows
        got = _AllToAllRows.apply(rows, send_l, recv_l, self.group)
        eid = torch.empty(sum(recv_l), dtype=torch.long, device=x.device)
        dist.all_to_all_single(eid, e_sorted - 0, output_split_sizes=recv_l, input_split_sizes=send_l, group=self.group)
        eid = eid - self.rank * self.El                               # local expert index of every received row
        if got.shape[0]:
            y = moe_ops.moe_mlp(got, torch.ones(got.shape[0], 1, dtype=torch.float32, device=x.device), eid.view(-1, 1),
                                gate_up_local, down_local)
        else:   # keep the local experts in the graph so that every rank runs the same backward collectives
            y = got + 0.0 * (gate_up_local.sum() + down_local.sum()).to(got.dtype)
        back = _AllToAllRows.apply(y, recv_l, send_l, self.group)     # expert outputs, in this rank's sorted pair order
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=order.device)
        per_pair = back.index_select(0, inv).view(M, k, D)
        return (per_pair.float() * w.float().unsqueeze(-1)).sum(1).to(x.dtype)
