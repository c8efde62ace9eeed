"""Micro-benchmarks of the fused compute + collective kernels (one process per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29520 -m omegalax_b200.parallel.microbench [--tokens 32768] [--iters 10]

For each fused path the device time (CUDA events, max over ranks, after warm-up) is reported
next to its unfused counterpart (own pull / NCCL collective + GEMM) and to its roofline: the
slower of FLOPs / measured GEMM peak and bytes that must cross NVLink / measured link rate.  The
GEMM peak is read from ``MEASURED_PEAKS.json`` at the repository root (``bf16_tflops``; 1590 if the
file is absent) and the link rate is measured at start-up with a peer copy of 256 MB from the next
rank (``--link-gbs`` overrides it).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops import lib
from . import symm

bf16 = torch.bfloat16
GEMM_PEAK_TFLOPS = 1590.0     # replaced by MEASURED_PEAKS.json when present (see _load_peaks)
LINK_GBS = 900.0              # nominal NVLink 5 per direction; replaced by the start-up measurement


def _load_peaks():
    global GEMM_PEAK_TFLOPS
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(os.path.dirname(os.path.dirname(here)), "MEASURED_PEAKS.json")
    try:
        GEMM_PEAK_TFLOPS = float(json.load(open(path)).get("bf16_tflops", GEMM_PEAK_TFLOPS))
        return "measured"
    except Exception:
        return "fallback"


def _measure_link(rank, world, dev, nbytes=256 << 20, iters=5):
    """Per-direction peer bandwidth: every rank pulls ``nbytes`` from its right neighbour with the
    pull all-gather kernel (all links busy at once, as in the collectives timed below)."""
    global LINK_GBS
    if world < 2:
        return LINK_GBS
    src = symm.SymmetricBuffer(nbytes)
    src.view(torch.uint8, nbytes).fill_(1)
    dst = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    tab = symm.make_copy_segments([((rank + 1) % world, 0, 0, nbytes)], dev)
    ms = _time(lambda: symm.allgather_pull(src, dst, tab), iters, 2, world)
    LINK_GBS = nbytes / ms / 1e6
    return LINK_GBS



def _time(fn, iters, warmup, world):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def _report(rank, name, ms, flops, link_bytes, **kw):
    if rank != 0:
        return
    t_c = flops / (GEMM_PEAK_TFLOPS * 1e9)
    t_l = link_bytes / (LINK_GBS * 1e6)
    roof = max(t_c, t_l)
    print(json.dumps({"path": name, "ms": round(ms, 4), "roofline_ms": round(roof, 4),
                      "bound": "compute" if t_c >= t_l else "nvlink", "fraction_of_roofline": round(roof / ms, 3),
                      **kw}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768, help="rows of the full activation matrix")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=24576, help="full output width of the gathered projections")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--link-gbs", type=float, default=None, help="link rate for the rooflines instead of measuring it")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    W = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if W > 1:
        dist.init_process_group("nccl", device_id=dev)
    bar = symm.DeviceBarrier() if W > 1 else (lambda: None)
    which = _load_peaks()
    global LINK_GBS
    if a.link_gbs:
        LINK_GBS = a.link_gbs
    else:
        _measure_link(rank, W, dev)
    if rank == 0:
        print(json.dumps({"gemm_peak_tflops": GEMM_PEAK_TFLOPS, "gemm_peak_source": which,
                          "link_gbs_per_direction": round(LINK_GBS, 1),
                          "link_source": "--link-gbs" if a.link_gbs else ("measured" if W > 1 else "nominal")}), flush=True)
    M, D, Fw = a.tokens, a.hidden, a.ffn
    m, f = M // W, Fw // W
    torch.manual_seed(rank)

    # ---- tensor parallel, column projection: all-gather rows of x -> GEMM with this rank's columns
    x_stage = symm.SymmetricBuffer(m * D * 2)
    x_stage.view(bf16, m * D).copy_(torch.randn(m * D, device=dev).to(bf16))
    w_col = torch.randn(f, D, device=dev).to(bf16)
    full = torch.empty(M, D, dtype=bf16, device=dev)
    flags = torch.zeros(W, dtype=torch.int32, device=dev)
    calls = [0]
    bar()

    c1 = K.ag_copy_ctas(M, f, D, W * m * D * 2.0)

    def fused_ag():
        calls[0] += c1
        K.gemm_ag(w_col, full, x_stage.peer_ptr_list(0), side=1, rank=rank, rows_per_rank=m, flags=flags,
                  target=calls[0], copy_ctas=c1)

    tab = symm.make_copy_segments([(r, 0, r * m * D * 2, m * D * 2) for r in range(W)], dev)

    def pull_then_gemm():
        symm.allgather_pull(x_stage, full, tab)
        K.gemm(full, w_col)

    xl = x_stage.view(bf16, m * D).view(m, D)

    def nccl_then_gemm():
        if W > 1:
            dist.all_gather_into_tensor(full, xl)
        K.gemm(full, w_col)

    fl = 2.0 * M * f * D
    link = (W - 1) * m * D * 2.0
    shape = dict(M=M, N=f, K=D, world=W)
    _report(rank, "TP column: all-gather(x) -> GEMM, one launch", _time(fused_ag, a.iters, a.warmup, W), fl, link,
            copy_ctas=c1, **shape)
    _report(rank, "  pull all-gather kernel, then GEMM", _time(pull_then_gemm, a.iters, a.warmup, W), fl, link, **shape)
    _report(rank, "  NCCL all_gather, then GEMM", _time(nccl_then_gemm, a.iters, a.warmup, W), fl, link, **shape)
    _report(rank, "  GEMM alone (operand already local)", _time(lambda: K.gemm(full, w_col), a.iters, a.warmup, W), fl, 0.0, **shape)

    # ---- FSDP: all-gather rows of W -> GEMM (weight chunks on the peers)
    n_full = 6144
    nr = n_full // W
    w_stage = symm.SymmetricBuffer(nr * D * 2)
    w_stage.view(bf16, nr * D).copy_(torch.randn(nr * D, device=dev).to(bf16))
    w_full = torch.empty(n_full, D, dtype=bf16, device=dev)
    x_full = torch.randn(M, D, device=dev).to(bf16)
    flags2 = torch.zeros(W, dtype=torch.int32, device=dev)
    calls2 = [0]
    bar()

    c2 = K.ag_copy_ctas(M, n_full, D, W * nr * D * 2.0)

    def fused_w():
        calls2[0] += c2
        K.gemm_ag(x_full, w_full, w_stage.peer_ptr_list(0), side=2, rank=rank, rows_per_rank=nr, flags=flags2,
                  target=calls2[0], copy_ctas=c2)

    fl2 = 2.0 * M * n_full * D
    link2 = (W - 1) * nr * D * 2.0
    if nr % 128 == 0:
        _report(rank, "FSDP: all-gather(W_qkv) -> GEMM, one launch", _time(fused_w, a.iters, a.warmup, W), fl2, link2,
                copy_ctas=c2, M=M, N=n_full, K=D, world=W)
        _report(rank, "  GEMM alone (weight already gathered)", _time(lambda: K.gemm(x_full, w_full), a.iters, a.warmup, W),
                fl2, 0.0, M=M, N=n_full, K=D, world=W)

    # ---- tensor parallel, row projection: GEMM -> reduce-scatter over rows in the epilogue
    h = torch.randn(M, max(512, 12288 // W), device=dev).to(bf16)              # [M, F/tp] activation slice
    w_row = torch.randn(D, h.shape[1], device=dev).to(bf16)
    rs = symm.SymmetricBuffer(m * D * 2)
    acc = rs.view(bf16, m * D)
    ptrs = rs.peer_ptr_list(0)

    def fused_rs():
        acc.zero_()
        bar()
        K.gemm_peer_reduce(h, w_row, ptrs, m, D, bf16_out=True)
        bar()

    y_full = torch.empty(M, D, dtype=bf16, device=dev)
    y_loc = torch.empty(m, D, dtype=bf16, device=dev)
    slabs = symm.SymmetricBuffer(W * m * D * 2)          # one [m, D] slab per sender on every owner
    slab_ptrs = slabs.peer_ptr_list(0)
    slab_view = slabs.view(bf16, W * m * D)

    def staged_rs():
        bar()                                            # the owner has summed the previous call's slabs
        K.gemm_peer_reduce(h, w_row, slab_ptrs, m, D, slot=rank)
        bar()
        K.slab_sum(slab_view, W, y_loc)

    def gemm_then_nccl():
        K.gemm(h, w_row, out=y_full)
        if W > 1:
            dist.reduce_scatter_tensor(y_loc, y_full)

    fl3 = 2.0 * M * D * h.shape[1]
    link3 = (W - 1) * m * D * 2.0
    _report(rank, "TP row: GEMM -> reduce-scatter in the epilogue (bf16 adds over NVLink, incl. clear + 2 barriers)",
            _time(fused_rs, a.iters, a.warmup, W), fl3, link3, M=M, N=D, K=h.shape[1], world=W)
    _report(rank, "TP row: GEMM -> per-sender slabs on the owner (plain stores over NVLink) -> slab sum (incl. 2 barriers)",
            _time(staged_rs, a.iters, a.warmup, W), fl3, link3, M=M, N=D, K=h.shape[1], world=W)
    _report(rank, "  GEMM, then NCCL reduce_scatter (bf16)", _time(gemm_then_nccl, a.iters, a.warmup, W), fl3,
            (W - 1) * m * D * 2.0, M=M, N=D, K=h.shape[1], world=W)

    # ---- expert parallel: dispatch push / combine pull against NCCL all_to_all of the same rows
    from .ep import ExpertParallel

    tok, topk, E, Dm = 16384, 8, 128, 2048
    if W > 1 and E % W == 0:
        ep = ExpertParallel(dist.group.WORLD, E, Dm, tok, topk, capacity_factor=2.0, reuse_buffers=True)
        xe = torch.randn(tok, Dm, device=dev).to(bf16)
        idx = torch.stack([torch.randperm(E, device=dev)[:topk] for _ in range(64)]).repeat(tok // 64, 1)
        wts = torch.full((tok, topk), 1.0 / topk, device=dev)
        from .ep import build_plan_device

        st = torch.arange(tok, device=dev, dtype=torch.int32).repeat_interleave(topk)
        plan = build_plan_device(idx, E, W, rank, dist.group.WORLD, ep.capacity, ep.overflow_flag, st)

        def disp():
            ep.barrier()
            ep.push(ep.buf_in, xe, plan)
            ep.barrier()

        def comb():
            ep.barrier()
            ep.pull(ep.buf_in, plan, weights=wts.reshape(-1))
            ep.barrier()

        rows = tok * topk
        send = torch.empty(rows, Dm, dtype=bf16, device=dev)
        recv = torch.empty(rows, Dm, dtype=bf16, device=dev)

        def nccl_a2a():
            dist.all_to_all_single(recv, send)

        link4 = rows * Dm * 2.0 * (W - 1) / W
        _report(rank, "EP dispatch: permute + all-to-all in one kernel (incl. 2 barriers)",
                _time(disp, a.iters, a.warmup, W), 0.0, link4, tokens=tok, top_k=topk, hidden=Dm, world=W)
        _report(rank, "EP combine: all-to-all + weighted un-permute in one kernel (incl. 2 barriers)",
                _time(comb, a.iters, a.warmup, W), 0.0, link4, tokens=tok, top_k=topk, hidden=Dm, world=W)
        _report(rank, "  NCCL all_to_all_single of the same rows (no permute)", _time(nccl_a2a, a.iters, a.warmup, W),
                0.0, link4, tokens=tok, top_k=topk, hidden=Dm, world=W)
        ep.check()
    torch.cuda.synchronize()
    lib.check_status()
    if W > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
