"""Kernel micro-benchmarks (one B200): device-timed with CUDA events after warm-up, with an L2
flush between timed launches, reported against the measured peaks of the box.

    python -m omegalax_b200.ops.microbench gemm --m 16384 --n 6144 --k 4096
    python -m omegalax_b200.ops.microbench attn --batch 8 --seq 4096 --heads 32 --kv-heads 8
    python -m omegalax_b200.ops.microbench gdn --batch 2 --seq 8192 --heads 64 --k-heads 16
    python -m omegalax_b200.ops.microbench decode --batch 32 --ctx 4096
    python -m omegalax_b200.ops.microbench elementwise --rows 32768 --cols 4096
    python -m omegalax_b200.ops.microbench ce --rows 8192 --vocab 151936

``--iters 0 --warmup N`` only launches the kernels N times (for a profiler capture of a small
case); ``--baseline`` also times the library counterpart (cuBLAS / SDPA) for comparison.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import kernels as K
from . import lib

bf16 = torch.bfloat16


def _peaks():
    here = os.path.dirname(os.path.abspath(__file__))
    p = os.path.join(os.path.dirname(os.path.dirname(here)), "MEASURED_PEAKS.json")
    try:
        d = json.load(open(p))
        return float(d.get("bf16_tflops", 1590.0)), float(d.get("hbm_gbs", 6650.0)), "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


def timeit(fn, iters: int, warmup: int, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if iters <= 0:
        return None
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.add_(1.0)           # 256 MB written: larger than L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def _report(name, ms, flops=None, bytes_=None, **extra):
    tf_peak, bw_peak, which = _peaks()
    out = {"kernel": name, "ms": ms, **extra}
    if ms:
        if flops:
            out["tflops"] = flops / ms / 1e9
            out[f"frac_of_{which}_bf16_burst"] = out["tflops"] / tf_peak
        if bytes_:
            out["gbs"] = bytes_ / ms / 1e6
            out[f"frac_of_{which}_hbm"] = out["gbs"] / bw_peak
    print(json.dumps(out), flush=True)


def bench_gemm(a, dev, flush):
    m, n, k = a.m, a.n, a.k
    x = torch.randn(m, k, device=dev).to(bf16)
    w = torch.randn(n, k, device=dev).to(bf16)
    dy = torch.randn(m, n, device=dev).to(bf16)
    acc = torch.zeros(n, k, device=dev)
    fl = 2.0 * m * n * k
    by = 2.0 * (m * k + n * k + m * n)
    _report("gemm fprop  y=x w^T", timeit(lambda: K.gemm(x, w), a.iters, a.warmup, flush), fl, by, m=m, n=n, k=k)
    _report("gemm dgrad  dx=dy w", timeit(lambda: K.gemm(dy, w, b_mn=True), a.iters, a.warmup, flush), fl, by, m=m, n=n, k=k)
    _report("gemm wgrad  dw+=dy^T x (fp32 accumulate)",
            timeit(lambda: K.gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True), a.iters, a.warmup, flush),
            fl, None, m=m, n=n, k=k)
    for nm, fn in (("fprop", lambda: K.gemm(x, w, pair=True)), ("dgrad", lambda: K.gemm(dy, w, b_mn=True, pair=True)),
                   ("wgrad fp32 accumulate", lambda: K.gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True, pair=True))):
        _report(f"gemm {nm}, CTA pairs (256x256 tiles)", timeit(fn, a.iters, a.warmup, flush), fl, None, m=m, n=n, k=k)
    if a.baseline:
        _report("cuBLAS fprop", timeit(lambda: torch.matmul(x, w.t()), a.iters, a.warmup, flush), fl, by)
        _report("cuBLAS dgrad", timeit(lambda: torch.matmul(dy, w), a.iters, a.warmup, flush), fl, by)
        _report("cuBLAS wgrad", timeit(lambda: torch.matmul(dy.t(), x), a.iters, a.warmup, flush), fl, None)


def bench_attn(a, dev, flush):
    B, T, H, G, HD = a.batch, a.seq, a.heads, a.kv_heads, a.head_dim
    q = torch.randn(B * T, H, HD, device=dev).to(bf16)
    k = torch.randn(B * T, G, HD, device=dev).to(bf16)
    v = torch.randn(B * T, G, HD, device=dev).to(bf16)
    do = torch.randn_like(q)
    cu = torch.arange(B + 1, device=dev, dtype=torch.int32) * T
    sc = HD ** -0.5
    o, lse = K.attn_fwd(q, k, v, cu, T, sc, True)
    fl = 4.0 * B * T * T * H * HD / 2
    _report("attention fwd (causal, GQA)", timeit(lambda: K.attn_fwd(q, k, v, cu, T, sc, True), a.iters, a.warmup, flush),
            fl, None, batch=B, seq=T, heads=H, kv_heads=G, head_dim=HD)
    if HD in (128, 256):
        _report("attention bwd (causal, GQA)",
                timeit(lambda: K.attn_bwd(q, k, v, o, lse, do, cu, T, sc, True), a.iters, a.warmup, flush), 2.5 * fl, None)
    if a.baseline:
        import torch.nn.functional as F

        q4, k4, v4 = (t.view(B, T, -1, HD).transpose(1, 2) for t in (q, k, v))
        _report("SDPA fwd", timeit(lambda: F.scaled_dot_product_attention(q4, k4, v4, is_causal=True, enable_gqa=True),
                                   a.iters, a.warmup, flush), fl, None)


def bench_gdn(a, dev, flush):
    B, T, H, Hk, A, U = a.batch, a.seq, a.heads, a.k_heads, 128, a.head_dim
    q = torch.nn.functional.normalize(torch.randn(B, T, Hk, A, device=dev), dim=-1) * A ** -0.5
    k = torch.nn.functional.normalize(torch.randn(B, T, Hk, A, device=dev), dim=-1)
    v = torch.randn(B, T, H, U, device=dev)
    g = -torch.rand(B, T, H, device=dev) * 0.3
    beta = torch.sigmoid(torch.randn(B, T, H, device=dev))
    do = torch.randn_like(v)
    o, n_out, states, _ = K.gdn_fwd(q, k, v, g, beta)
    J = T // 64
    macs_f = B * H * J * (2 * 64 * 64 * A + 2 * 64 * A * U + 64 * 64 * U + A * 64 * U)
    _report("gated delta rule fwd (fp32)", timeit(lambda: K.gdn_fwd(q, k, v, g, beta), a.iters, a.warmup, flush),
            2.0 * macs_f, None, batch=B, seq=T, heads=H, k_heads=Hk, head_dim_v=U)
    _report("gated delta rule bwd (fp32)",
            timeit(lambda: K.gdn_bwd(q, k, v, g, beta, n_out, states, do), a.iters, a.warmup, flush), None, None)
    x = torch.randn(B, T, 2 * Hk * A + H * U, device=dev).to(bf16)
    w = torch.randn(x.shape[-1], 4, device=dev).to(bf16)
    by = 2.0 * x.numel() * 2
    _report("causal conv1d+SiLU fwd", timeit(lambda: K.causal_conv1d_fwd(x, w), a.iters, a.warmup, flush), None, by)
    dw = torch.zeros(w.shape, device=dev)
    _report("causal conv1d+SiLU bwd", timeit(lambda: K.causal_conv1d_bwd(x, w, x, dw), a.iters, a.warmup, flush), None, 1.5 * by)


def bench_decode(a, dev, flush):
    B, H, G, HD, ctx, page = a.batch, a.heads, a.kv_heads, 128, a.ctx, 64
    blocks = -(-(ctx + 1) // page)
    k_pages = torch.randn(B * blocks, page, G, HD, device=dev).to(bf16)
    v_pages = torch.randn(B * blocks, page, G, HD, device=dev).to(bf16)
    table = torch.randperm(B * blocks, device=dev).to(torch.int32).view(B, blocks)
    lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    q = torch.randn(B, H, HD, device=dev).to(bf16)
    by = 2.0 * B * ctx * G * HD * 2
    _report("paged decode attention (split-KV, GQA)",
            timeit(lambda: K.decode_attn(q, k_pages, v_pages, table, lens, page, HD ** -0.5), a.iters, a.warmup, flush),
            None, by, batch=B, ctx=ctx, heads=H, kv_heads=G)


def bench_elementwise(a, dev, flush):
    M, D = a.rows, a.cols
    x = torch.randn(M, D, device=dev).to(bf16)
    w = torch.ones(D, device=dev).to(bf16)
    by = 2.0 * M * D * 2
    _report("rmsnorm fwd", timeit(lambda: K.rmsnorm_fwd(x, w, 1e-6), a.iters, a.warmup, flush), None, by, rows=M, cols=D)
    H, G, Kd = 32, 8, 128
    qkv = torch.randn(M, (H + 2 * G) * Kd, device=dev).to(bf16)
    qw, kw = torch.ones(Kd, device=dev).to(bf16), torch.ones(Kd, device=dev).to(bf16)
    ang = torch.rand(M, Kd // 2, device=dev) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    q, k = K.qknorm_rope_fwd(qkv, qw, kw, cos, sin, H, G, Kd, Kd, 1e-6)
    qb = 2.0 * M * (H + G) * Kd * 2
    _report("qk-norm + rope fwd", timeit(lambda: K.qknorm_rope_fwd(qkv, qw, kw, cos, sin, H, G, Kd, Kd, 1e-6),
                                         a.iters, a.warmup, flush), None, qb, rows=M, heads=H, kv_heads=G)
    dqkv = torch.zeros_like(qkv)
    dqw, dkw = torch.zeros(Kd, device=dev), torch.zeros(Kd, device=dev)
    _report("qk-norm + rope bwd",
            timeit(lambda: K.qknorm_rope_bwd(qkv, qw, kw, cos, sin, q, k, dqkv, dqw, dkw, H, G, Kd, Kd, 1e-6),
                   a.iters, a.warmup, flush), None, 1.5 * qb)
    gu = torch.randn(M, 2 * D, device=dev).to(bf16)
    _report("swiglu fwd", timeit(lambda: K.swiglu_fwd(gu), a.iters, a.warmup, flush), None, 3.0 * M * D * 2)


def bench_ce(a, dev, flush):
    from . import functional as Fn

    M, V, D = a.rows, a.vocab, a.cols
    h = (torch.randn(M, D, device=dev) * 0.5).to(bf16).requires_grad_(True)
    w = (torch.randn(V, D, device=dev) * 0.02).to(bf16).requires_grad_(True)
    y = torch.randint(0, V, (M,), device=dev)
    mask = torch.ones(M, device=dev)

    def step():
        loss = Fn.linear_cross_entropy(h, w, y.to(torch.int32), mask, 1.0 / M)
        loss.backward()
        h.grad = None
        w.grad = None

    _report("fused linear + cross-entropy fwd+bwd", timeit(step, a.iters, a.warmup, flush), 6.0 * M * V * D, None,
            rows=M, vocab=V, hidden=D)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attn", "gdn", "decode", "elementwise", "ce"])
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--k-heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--baseline", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.zeros(64 * 1024 * 1024, device=dev) if a.iters > 0 else None
    {"gemm": bench_gemm, "attn": bench_attn, "gdn": bench_gdn, "decode": bench_decode,
     "elementwise": bench_elementwise, "ce": bench_ce}[a.what](a, dev, flush)
    torch.cuda.synchronize()
    lib.check_status()


if __name__ == "__main__":
    main()
