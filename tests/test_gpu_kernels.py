"""Each sm_100a kernel against a plain PyTorch fp32 evaluation of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

bf16 = torch.bfloat16


def _dev():
    return torch.device("cuda", 0)


def _check(lib):
    torch.cuda.synchronize()
    lib.check_status()


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).abs().max() / (b.abs().max() + 1e-6))


def _assert_gemm_close(out, ref, K):
    """Per-element check with tolerances true to the output type: a bf16 result may differ from the
    fp32 reference by 2 ulp (2^-7 relative), an fp32 result by 1e-4; the absolute term covers sums
    that cancel (terms of size ~1, K of them, fp32 accumulation in a different order)."""
    if out.dtype == bf16:
        torch.testing.assert_close(out.float(), ref, rtol=2.0 ** -7, atol=2.0 ** -7 * math.sqrt(K) * 0.25)
    else:
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=2e-5 * math.sqrt(K))


@pytest.mark.parametrize("M,N,K", [(512, 512, 256), (304, 520, 136), (1000, 776, 4160)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("mode", ["bf16", "fp32", "acc"])
@pytest.mark.parametrize("wide", [0, 1])
def test_gemm_pair_every_output_mode_per_element(M, N, K, a_mn, b_mn, mode, wide):
    """CTA-pair kernels (256 x 256 tile, and the 512 x 256 tile one with its TMA-store epilogue) on
    shapes that are not multiples of the tile, every output mode, checked element by element
    against fp32 matmul of the same bf16 inputs."""
    from omegalax_b200.ops import kernels as Kn, lib
    torch.manual_seed(10)
    lib.gemm_pair_tune(-1, wide, -1)
    a = torch.randn(M, K, device=_dev()).to(bf16)
    b = torch.randn(N, K, device=_dev()).to(bf16)
    ref = a.float() @ b.float().t()
    aa = a.t().contiguous() if a_mn else a
    bb = b.t().contiguous() if b_mn else b
    if mode == "bf16":
        out = Kn.gemm(aa, bb, a_mn=a_mn, b_mn=b_mn, pair=True)
    elif mode == "fp32":
        out = Kn.gemm(aa, bb, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, pair=True)
    else:
        out = torch.full((M, N), 0.5, device=_dev(), dtype=torch.float32)
        Kn.gemm(aa, bb, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=True, pair=True)
        ref = ref + 0.5
    lib.gemm_pair_tune(-1, -1, -1)
    _check(lib)
    _assert_gemm_close(out, ref, K)


@pytest.mark.parametrize("wide", [0, 1])
@pytest.mark.parametrize("splits", [-1, 1, 2, 3, 8])
def test_gemm_pair_split_reduction(splits, wide):
    """Weight-gradient layout with a long reduction: the (tile, slice) units of the split reduction
    add up to the unsplit result; -1 lets the launcher choose (few tiles -> it splits)."""
    from omegalax_b200.ops import kernels as Kn, lib
    torch.manual_seed(11)
    M, N, K = 512, 768, 8192 + 64      # 6 tiles; K not a multiple of the slice length
    dy = torch.randn(K, M, device=_dev()).to(bf16)
    x = torch.randn(K, N, device=_dev()).to(bf16)
    ref = dy.float().t() @ x.float() + 1.0
    lib.gemm_pair_tune(-1, wide, splits)
    try:
        out = torch.ones(M, N, device=_dev(), dtype=torch.float32)
        Kn.gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=True, pair=True)
        _check(lib)
    finally:
        lib.gemm_pair_tune(-1, -1, -1)
    _assert_gemm_close(out, ref, K)


@pytest.mark.parametrize("wide", [0, 1])
def test_gemm_pair_unaligned_output_pitch_and_local_peer_reduce(wide):
    """Outputs the TMA unit cannot address (row pitch not a multiple of 16 bytes) take the
    register -> global path; the peer-reduction epilogue is exercised with both "peers" being
    buffers of this GPU (row blocks of the result land in two separate allocations)."""
    from omegalax_b200.ops import kernels as Kn, lib
    torch.manual_seed(13)
    M, N, K = 1024, 520, 2048 + 64
    a = torch.randn(M, K, device=_dev()).to(bf16)
    b = torch.randn(N, K, device=_dev()).to(bf16)
    ref = a.float() @ b.float().t()
    big = torch.zeros(M, N + 4, device=_dev(), dtype=bf16)
    big32 = torch.full((M, N + 1), 2.0, device=_dev(), dtype=torch.float32)
    lib.gemm_pair_tune(-1, wide, -1)
    try:
        Kn.gemm(a, b, out=big[:, :N], pair=True)
        Kn.gemm(a, b, out=big32[:, :N], accumulate=True, pair=True)
        halves = [torch.zeros(M // 2, N, device=_dev(), dtype=torch.float32) for _ in range(2)]
        Kn.gemm_peer_reduce(a, b, [h.data_ptr() for h in halves], M // 2, N, pair=True)
        Kn.gemm_peer_reduce(a, b, [h.data_ptr() for h in halves], M // 2, N, pair=True)
        _check(lib)
    finally:
        lib.gemm_pair_tune(-1, -1, -1)
    _assert_gemm_close(big[:, :N], ref, K)
    assert float(big[:, N:].abs().max()) == 0.0          # nothing written beyond the view
    _assert_gemm_close(big32[:, :N].contiguous(), ref + 2.0, K)
    assert float((big32[:, N:] - 2.0).abs().max()) == 0.0
    _assert_gemm_close(torch.cat(halves, 0), 2 * ref, K)


@pytest.mark.parametrize("pair", [False, True])
def test_gemm_peer_reduce_starting_at_another_owner(pair):
    """The tile rows may be walked starting at any owner's block (each GPU of a group starts at its
    own): every row block is still produced exactly once."""
    from omegalax_b200.ops import kernels as Kn, lib
    from omegalax_b200.parallel.symm import PeerPtrs
    torch.manual_seed(14)
    M, N, K, W = 2048 + 256, 384, 512, 4      # 576 rows per owner: not a multiple of the tile height
    a = torch.randn(K, M, device=_dev()).to(bf16)
    b = torch.randn(K, N, device=_dev()).to(bf16)
    ref = a.float().t() @ b.float()
    for first in range(W):
        parts = [torch.zeros(M // W, N, device=_dev()) for _ in range(W)]
        ptrs = PeerPtrs(t.data_ptr() for t in parts)
        ptrs.rank = first
        Kn.gemm_peer_reduce(a, b, ptrs, M // W, N, a_mn=True, b_mn=True, pair=pair)
        _check(lib)
        _assert_gemm_close(torch.cat(parts, 0), ref, K)


@pytest.mark.parametrize("kernel", ["single", "pair", "wide"])
def test_gemm_two_phase_reduce_scatter_on_local_slabs(kernel):
    """First phase: two "senders" (two GEMMs with different operands) store their bf16 result rows
    into their own slab of each owner's staging buffer; second phase: every owner sums its slabs
    and adds the residual.  Both owners are buffers of this GPU."""
    from omegalax_b200.ops import kernels as Kn, lib
    torch.manual_seed(18)
    M, N, K, W = 1024, 520, 320, 2
    m = M // W
    xs = [torch.randn(M, K, device=_dev()).to(bf16) for _ in range(W)]
    ws = [torch.randn(N, K, device=_dev()).to(bf16) for _ in range(W)]
    res = torch.randn(M, N, device=_dev()).to(bf16)
    stage = [torch.full((W, m, N), float("nan"), device=_dev(), dtype=bf16) for _ in range(W)]   # per owner
    lib.gemm_pair_tune(-1, 1 if kernel == "wide" else 0, -1)
    try:
        for sender in range(W):
            Kn.gemm_peer_reduce(xs[sender], ws[sender], [t.data_ptr() for t in stage], m, N, slot=sender,
                                pair=kernel != "single")
        outs = [Kn.slab_sum(stage[o], W, torch.empty(m, N, device=_dev(), dtype=bf16), res[o * m:(o + 1) * m].contiguous())
                for o in range(W)]
        _check(lib)
    finally:
        lib.gemm_pair_tune(-1, -1, -1)
    parts = [(xs[s].float() @ ws[s].float().t()).to(bf16).float() for s in range(W)]    # each slab is rounded to bf16
    ref = parts[0] + parts[1] + res.float()
    torch.testing.assert_close(torch.cat(outs, 0).float(), ref, rtol=2.0 ** -7, atol=0.15)


@pytest.mark.parametrize("gm,wide", [(2, 0), (16, 0), (3, 1), (16, 1)])
def test_gemm_pair_raster_knob(gm, wide):
    from omegalax_b200.ops import kernels as Kn, lib
    torch.manual_seed(12)
    M, N, K = 2304, 1280, 1024 + 64
    a = torch.randn(M, K, device=_dev()).to(bf16)
    b = torch.randn(N, K, device=_dev()).to(bf16)
    ref = a.float() @ b.float().t()
    lib.gemm_pair_tune(gm, wide, -1)
    try:
        out = Kn.gemm(a, b, pair=True)
        out_t = Kn.gemm(a, b.t().contiguous(), b_mn=True, pair=True)
        _check(lib)
    finally:
        lib.gemm_pair_tune(-1, -1, -1)
    _assert_gemm_close(out, ref, K)
    _assert_gemm_close(out_t, ref, K)


@pytest.mark.parametrize("M,N,K", [(256, 512, 384), (300, 200, 136), (1024, 1024, 1024), (128, 4096, 64), (4096, 1536, 2048)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    from omegalax_b200.ops import kernels as Kn, lib
    torch.manual_seed(0)
    if a_mn and M % 8:
        pytest.skip("MN-major A needs a 16-byte aligned M pitch")
    if b_mn and N % 8:
        pytest.skip("MN-major B needs a 16-byte aligned N pitch")
    a = torch.randn(M, K, device=_dev()).to(bf16)
    b = torch.randn(N, K, device=_dev()).to(bf16)
    ref = a.float() @ b.float().t()
    aa = a.t().contiguous() if a_mn else a
    bb = b.t().contiguous() if b_mn else b
    out = Kn.gemm(aa, bb, a_mn=a_mn, b_mn=b_mn)
    _check(lib)
    assert out.shape == (M, N)
    assert _rel_err(out, ref) < 2e-2


@pytest.mark.parametrize("kernel", ["single", "pair", "wide"])
@pytest.mark.parametrize("with_res", [False, True])
def test_gemm_bias_epilogue(kernel, with_res):
    """y = x W^T + bias (+ residual) in the GEMM epilogue, on every GEMM kernel, per element."""
    from omegalax_b200.ops import kernels as Kn, lib
    torch.manual_seed(14)
    M, N, K = 776, 328, 192
    a = torch.randn(M, K, device=_dev()).to(bf16)
    b = torch.randn(N, K, device=_dev()).to(bf16)
    bias = torch.randn(N, device=_dev()).to(bf16)
    res = torch.randn(M, N, device=_dev()).to(bf16) if with_res else None
    ref = a.float() @ b.float().t() + bias.float() + (res.float() if with_res else 0.0)
    lib.gemm_pair_tune(-1, 1 if kernel == "wide" else 0, -1)
    try:
        out = Kn.gemm(a, b, bias=bias, residual=res, pair=kernel != "single")
        _check(lib)
    finally:
        lib.gemm_pair_tune(-1, -1, -1)
    _assert_gemm_close(out, ref, K)


def test_linear_with_bias_gradients():
    from omegalax_b200.ops import functional as Fn, lib
    torch.manual_seed(15)
    x = torch.randn(3, 100, 256, device=_dev()).to(bf16).requires_grad_(True)
    w = (torch.randn(384, 256, device=_dev()) * 0.05).to(bf16).requires_grad_(True)
    b = torch.randn(384, device=_dev()).to(bf16).requires_grad_(True)
    r = torch.randn(3, 100, 384, device=_dev()).to(bf16).requires_grad_(True)
    y = Fn.linear(x, w, residual=r, bias=b)
    dy = torch.randn_like(y)
    y.backward(dy)
    _check(lib)
    xr, wr, br, rr = (t.detach().float().requires_grad_(True) for t in (x, w, b, r))
    yr = torch.nn.functional.linear(xr, wr, br) + rr
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, rtol=2.0 ** -7, atol=0.05)
    for got, want in ((x.grad, xr.grad), (w.grad, wr.grad), (b.grad, br.grad), (r.grad, rr.grad)):
        assert _rel_err(got, want) < 1e-2


@pytest.mark.parametrize("V", [1024, 151936 // 8 + 8, 5000 - 8])
def test_linear_cross_entropy_loss_is_that_of_fp32_logits(V):
    """The loss comes from the fp32 accumulator of the logits GEMM (statistics epilogue), not from
    bf16-rounded logits: it equals the fp32 PyTorch value to 1e-5 relative; the gradients, which
    go through bf16 dlogits, to bf16 accuracy."""
    from omegalax_b200.ops import functional as Fn, lib
    torch.manual_seed(16)
    M, D = 600, 256
    h = torch.randn(M, D, device=_dev()).to(bf16).requires_grad_(True)
    w = (torch.randn(V, D, device=_dev()) * 0.1).to(bf16).requires_grad_(True)
    y = torch.randint(0, V, (M,), device=_dev(), dtype=torch.int32)
    mask = (torch.rand(M, device=_dev()) > 0.3).float()
    loss = Fn.linear_cross_entropy(h, w, y, mask, 1.0 / M, chunk=256)
    loss.backward()
    _check(lib)
    hr, wr = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    logits = hr @ wr.t()
    nll = torch.nn.functional.cross_entropy(logits, y.long(), reduction="none")
    ref = (nll * mask).sum() / M
    ref.backward()
    assert abs(float(loss) - float(ref)) <= 1e-5 * abs(float(ref)) + 1e-6, (float(loss), float(ref))
    # the gradients go through the bf16 copy of the logits (off by up to 2^-9 relative)
    assert _rel_err(h.grad, hr.grad) < 3e-2
    assert _rel_err(w.grad, wr.grad) < 3e-2


@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_epilogues(bn):
    from omegalax_b200.ops import kernels as Kn, lib
    torch.manual_seed(1)
    M, N, K = 384, 640, 256
    a = torch.randn(M, K, device=_dev()).to(bf16)
    b = torch.randn(N, K, device=_dev()).to(bf16)
    res = torch.randn(M, N, device=_dev()).to(bf16)
    ref = a.float() @ b.float().t()
    out = Kn.gemm(a, b, residual=res, bn=bn)
    _check(lib)
    assert _rel_err(out, ref + res.float()) < 2e-2
    acc = torch.ones(M, N, device=_dev(), dtype=torch.float32)
    Kn.gemm(a, b, out=acc, accumulate=True, bn=bn)
    Kn.gemm(a, b, out=acc, accumulate=True, bn=bn)
    _check(lib)
    assert _rel_err(acc, 2 * ref + 1) < 1e-2
    o32 = Kn.gemm(a, b, out_dtype=torch.float32, bn=bn)
    _check(lib)
    assert _rel_err(o32, ref) < 1e-2


@pytest.mark.parametrize("pair", [False, True])
def test_gemm_grouped_and_wgrad(pair):
    """Grouped expert GEMMs (forward, input gradient, weight gradient) on the single-CTA kernel
    (segments padded to 128 rows) and on CTA pairs (segments padded to 256 rows; one expert is left
    empty), per expert against fp32 matmul."""
    from omegalax_b200.ops import kernels as Kn, lib
    from omegalax_b200.ops import moe
    torch.manual_seed(2)
    E, D, F, M, k = 5, 256, 384, 700, 2
    idx = torch.randint(0, E - 1, (M, k), device=_dev())      # expert E-1 receives nothing
    dest, offsets, cap = moe.build_permutation(idx, E, pad=256 if pair else 128)
    x = torch.randn(M, D, device=_dev()).to(bf16)
    xp = torch.zeros(cap, D, device=_dev(), dtype=bf16)
    tok = torch.arange(M, device=_dev()).repeat_interleave(k)
    xp.index_copy_(0, dest, x[tok])
    w = torch.randn(E, F, D, device=_dev()).to(bf16) * 0.05
    y = Kn.gemm_grouped(xp, w, offsets, pair=pair)
    _check(lib)
    offs = offsets.tolist()
    if pair:
        assert all(o % 256 == 0 for o in offs) and cap % 256 == 0
    for e in range(E):
        a, b = offs[e], offs[e + 1]
        if b > a:
            _assert_gemm_close(y[a:b], xp[a:b].float() @ w[e].float().t(), D)
    # dgrad layout: B given as [E, K, N]
    wt = w.transpose(1, 2).contiguous()
    y2 = Kn.gemm_grouped(xp, wt, offsets, b_mn=True, pair=pair)
    _check(lib)
    torch.testing.assert_close(y2[: offs[-1]].float(), y[: offs[-1]].float(), rtol=2.0 ** -7, atol=2e-2)
    dy = torch.randn(cap, F, device=_dev()).to(bf16)
    dw = torch.full((E, F, D), 0.25, device=_dev(), dtype=torch.float32)
    Kn.gemm_grouped_wgrad(dy, xp, offsets, dw, accumulate=True, pair=pair)
    _check(lib)
    for e in range(E):
        a, b = offs[e], offs[e + 1]
        ref = dy[a:b].float().t() @ xp[a:b].float() + 0.25
        _assert_gemm_close(dw[e], ref, max(b - a, 1))


@pytest.mark.parametrize("D", [64, 1024, 4096])
@pytest.mark.parametrize("one_plus", [False, True])
def test_rmsnorm(D, one_plus):
    from omegalax_b200.ops import functional as Fn, reference as R, lib
    torch.manual_seed(3)
    x = torch.randn(70, D, device=_dev()).to(bf16).requires_grad_(True)
    w = (torch.randn(D, device=_dev()) * 0.1 + (0 if one_plus else 1)).to(bf16).requires_grad_(True)
    y = Fn.rmsnorm(x, w, 1e-6, one_plus)
    dy = torch.randn_like(y)
    y.backward(dy)
    _check(lib)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = R.rmsnorm(xr, wr, 1e-6, one_plus)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 2e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2


def test_swiglu():
    from omegalax_b200.ops import functional as Fn, reference as R, lib
    torch.manual_seed(4)
    gu = torch.randn(100, 512, device=_dev()).to(bf16).requires_grad_(True)
    y = Fn.swiglu(gu)
    dy = torch.randn_like(y)
    y.backward(dy)
    _check(lib)
    gr = gu.detach().float().requires_grad_(True)
    yr = R.swiglu(gr)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(gu.grad, gr.grad) < 2e-2


@pytest.mark.parametrize("with_res,leaf", [(False, True), (True, True), (True, False)])
def test_swiglu_linear_keeps_only_gate_up(with_res, leaf):
    """silu(gate) * up followed by the down projection as one autograd node: the activation is not
    kept, its copy for the weight gradient comes out of the SwiGLU backward kernel.  A non-leaf
    [gate | up] (the usual case: a projection's output) receives its gradient in place."""
    from omegalax_b200.ops import functional as Fn, lib
    torch.manual_seed(41)
    M, Fh, D = 300, 256, 136
    gu0 = (0.7 * torch.randn(M, 2 * Fh, device=_dev())).to(bf16).requires_grad_(True)
    gu = gu0 if leaf else gu0 * 1.0
    ptr = gu.data_ptr()
    w = (torch.randn(D, Fh, device=_dev()) / 16).to(bf16).requires_grad_(True)
    res = torch.randn(M, D, device=_dev()).to(bf16).requires_grad_(True) if with_res else None
    y = Fn.swiglu_linear(gu, w, res)
    dy = torch.randn_like(y)
    y.backward(dy)
    _check(lib)
    gr, wr = gu0.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    act = torch.nn.functional.silu(gr[:, :Fh]) * gr[:, Fh:]
    yr = act.to(bf16).float() @ wr.t()          # the kernel path rounds the activation to bf16 too
    if with_res:
        rr = res.detach().float().requires_grad_(True)
        yr = yr + rr
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, rtol=2.0 ** -7, atol=2e-2)
    torch.testing.assert_close(gu0.grad.float(), gr.grad, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=2e-2, atol=6e-2)
    if with_res:
        assert torch.equal(res.grad, dy)
    if not leaf:      # the gradient was written over the (dead) input, not into a new buffer
        assert torch.equal(gu.detach().view(-1)[:64], gu0.grad.view(-1)[:64]) and gu.data_ptr() == ptr


@pytest.mark.parametrize("Kd,rot,qs", [(128, 128, 1), (64, 64, 1), (256, 64, 2)])
def test_qknorm_rope(Kd, rot, qs):
    from omegalax_b200.ops import functional as Fn, reference as R, lib
    torch.manual_seed(5)
    M, H, G = 96, 4, 2
    qkv = torch.randn(M, (H * qs + 2 * G) * Kd, device=_dev()).to(bf16).requires_grad_(True)
    qw = (1 + 0.1 * torch.randn(Kd, device=_dev())).to(bf16).requires_grad_(True)
    kw = (1 + 0.1 * torch.randn(Kd, device=_dev())).to(bf16).requires_grad_(True)
    sin, cos = R.rope_tables(torch.arange(M, device=_dev()), rot, 1e6)
    q, k, v, gate = Fn.qk_norm_rope(qkv, qw, kw, sin, cos, H, G, Kd, rot=rot, q_stride_heads=qs)
    dq, dk = torch.randn_like(q), torch.randn_like(k)
    torch.autograd.backward([q, k], [dq, dk])
    _check(lib)
    import os
    os.environ["OMEGALAX_B200_REFERENCE_OPS"] = "1"
    try:
        qkv_r = qkv.detach().float().requires_grad_(True)
        qw_r, kw_r = qw.detach().float().requires_grad_(True), kw.detach().float().requires_grad_(True)
        qr, kr, vr, _ = Fn.qk_norm_rope(qkv_r, qw_r, kw_r, sin, cos, H, G, Kd, rot=rot, q_stride_heads=qs)
        torch.autograd.backward([qr, kr], [dq.float(), dk.float()])
    finally:
        del os.environ["OMEGALAX_B200_REFERENCE_OPS"]
    assert _rel_err(q, qr) < 2e-2 and _rel_err(k, kr) < 2e-2
    assert _rel_err(qkv.grad, qkv_r.grad) < 3e-2
    assert _rel_err(qw.grad, qw_r.grad) < 3e-2 and _rel_err(kw.grad, kw_r.grad) < 3e-2


@pytest.mark.parametrize("HD", [128, 64])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("T", [128, 384, 1000])
def test_attention_forward(HD, causal, T):
    from omegalax_b200.ops import kernels as Kn, reference as R, lib
    torch.manual_seed(6)
    B, H, G = 2, 4, 2
    q = torch.randn(B * T, H, HD, device=_dev()).to(bf16)
    k = torch.randn(B * T, G, HD, device=_dev()).to(bf16)
    v = torch.randn(B * T, G, HD, device=_dev()).to(bf16)
    cu = torch.arange(B + 1, device=_dev(), dtype=torch.int32) * T
    scale = HD ** -0.5
    o, lse = Kn.attn_fwd(q, k, v, cu, T, scale, causal)
    _check(lib)
    ref = R.attention(q.view(B, T, H, HD).float(), k.view(B, T, G, HD).float(), v.view(B, T, G, HD).float(),
                      causal=causal, scale=scale).reshape(B * T, H, HD)
    assert _rel_err(o, ref) < 2e-2


def test_attention_varlen_strided_v():
    from omegalax_b200.ops import kernels as Kn, reference as R, lib
    torch.manual_seed(7)
    H, G, HD = 4, 2, 128
    lens = [200, 456, 77]
    N = sum(lens)
    qkv = torch.randn(N, (H + 2 * G) * HD, device=_dev()).to(bf16)
    q = qkv[:, : H * HD].reshape(N, H, HD).contiguous()
    k = qkv[:, H * HD:(H + G) * HD].reshape(N, G, HD).contiguous()
    v = qkv[:, (H + G) * HD:].view(N, G, HD)
    cu = torch.tensor([0, 200, 656, 733], device=_dev(), dtype=torch.int32)
    o, _ = Kn.attn_fwd(q, k, v, cu, max(lens), HD ** -0.5, True)
    _check(lib)
    ref = R.attention_varlen(q.float(), k.float(), v.float(), cu, causal=True, scale=HD ** -0.5)
    assert _rel_err(o, ref) < 2e-2


def test_linear_cross_entropy():
    from omegalax_b200.ops import functional as Fn, lib
    torch.manual_seed(8)
    M, D, V = 300, 256, 2048
    h = (torch.randn(M, D, device=_dev()) * 0.5).to(bf16).requires_grad_(True)
    w = (torch.randn(V, D, device=_dev()) * 0.05).to(bf16).requires_grad_(True)
    tgt = torch.randint(0, V, (M,), device=_dev())
    mask = (torch.rand(M, device=_dev()) > 0.5).float()
    scale = 1.0 / mask.sum()
    loss = Fn.linear_cross_entropy(h, w, tgt, mask, scale, chunk=128)
    loss.backward()
    _check(lib)
    hr = h.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    lr = Fn.linear_cross_entropy(hr, wr, tgt, mask, scale, chunk=128)
    lr.backward()
    assert abs(float(loss) - float(lr)) < 2e-2 * abs(float(lr))
    assert _rel_err(h.grad, hr.grad) < 3e-2
    assert _rel_err(w.grad, wr.grad) < 3e-2


def test_embedding_and_optimizer_kernels():
    from omegalax_b200.ops import kernels as Kn, lib
    torch.manual_seed(9)
    V, D, M = 512, 128, 300
    table = torch.randn(V, D, device=_dev()).to(bf16)
    ids = torch.randint(0, V, (M,), device=_dev())
    out = Kn.embedding_fwd(ids, table)
    assert torch.equal(out, table[ids])
    dy = torch.randn(M, D, device=_dev()).to(bf16)
    dt = torch.zeros(V, D, device=_dev())
    Kn.embedding_bwd(ids, dy, dt)
    ref = torch.zeros(V, D, device=_dev()).index_add_(0, ids, dy.float())
    _check(lib)
    assert _rel_err(dt, ref) < 1e-5
    # the same gradient with the table's rows split over four owners (here four buffers of one GPU)
    shards = [torch.zeros(V // 4, D, device=_dev()) for _ in range(4)]
    Kn.embedding_bwd_peer(ids, dy, [t.data_ptr() for t in shards], V // 4)
    _check(lib)
    assert _rel_err(torch.cat(shards), ref) < 1e-5
    n = 100003
    p = torch.randn(n, device=_dev()); m = torch.zeros(n, device=_dev()); v = torch.zeros(n, device=_dev())
    g = torch.randn(n, device=_dev()); p16 = torch.empty(n, device=_dev(), dtype=bf16)
    nsq = torch.zeros(1, device=_dev())
    Kn.sumsq(g, nsq)
    _check(lib)
    assert abs(float(nsq) - float((g.double() ** 2).sum())) < 1e-3 * float(nsq)
    p0, g0 = p.clone(), g.clone()
    Kn.adamw(p, m, v, g, p16, lr=1e-2, b1=0.9, b2=0.999, eps=1e-8, wd=0.01, step=1, grad_mul=0.5,
             norm_sq=nsq, max_norm=1.0)
    _check(lib)
    mul = 0.5 * min(1.0, 1.0 / (math.sqrt(float(nsq)) * 0.5 + 1e-6))
    gg = g0 * mul
    mr = 0.1 * gg
    vr = 0.001 * gg * gg
    pr = p0 - 1e-2 * ((mr / 0.1) / ((vr / 0.001).sqrt() + 1e-8) + 0.01 * p0)
    assert _rel_err(p, pr) < 1e-5
    assert float(g.abs().max()) == 0.0
    assert _rel_err(p16, pr) < 1e-2


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("T,B", [(256, 2), (1000, 2), (77, 3)])
def test_attention_backward(causal, T, B):
    from omegalax_b200.ops import kernels as Kn, reference as R, lib
    torch.manual_seed(10)
    H, G, HD = 4, 2, 128
    N = B * T
    q = torch.randn(N, H, HD, device=_dev()).to(bf16)
    k = torch.randn(N, G, HD, device=_dev()).to(bf16)
    v = torch.randn(N, G, HD, device=_dev()).to(bf16)
    do = torch.randn(N, H, HD, device=_dev()).to(bf16)
    cu = torch.arange(B + 1, device=_dev(), dtype=torch.int32) * T
    scale = HD ** -0.5
    o, lse = Kn.attn_fwd(q, k, v, cu, T, scale, causal)
    dq, dk, dv = Kn.attn_bwd(q, k, v, o, lse, do, cu, T, scale, causal)
    _check(lib)
    qr, kr, vr = (t.float().view(B, T, -1, HD).requires_grad_(True) for t in (q, k, v))
    ref = R.attention(qr, kr, vr, causal=causal, scale=scale)
    ref.backward(do.float().view(B, T, H, HD))
    assert _rel_err(dq, qr.grad.reshape(N, H, HD)) < 3e-2
    assert _rel_err(dk, kr.grad.reshape(N, G, HD)) < 3e-2
    assert _rel_err(dv, vr.grad.reshape(N, G, HD)) < 3e-2


def test_paged_decode_matches_full_forward():
    """Prefill a left-padded batch into the paged cache, then decode 6 steps with the paged
    kernels; every step's logits must agree with a full forward over the grown sequence."""
    import dataclasses

    from omegalax_b200.ops import lib
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.text import api as text_api

    mesh_lib.set_default_mesh(None)
    cfg = dataclasses.replace(text_api.resolve_config("Qwen/Qwen3-8B"), num_layers=2, emb_dim=256, mlp_dim=512,
                              num_heads=4, num_kv_heads=2, vocab_size=1024)
    model, cfg = text_api.init_model(cfg, 0, tp_size=1, fsdp_size=1, dp_size=1, device=_dev(), dtype=bf16)
    torch.manual_seed(0)
    B, T = 3, 40
    tok = torch.randint(1, 1024, (B, T), device=_dev())
    tok[1, :7] = 0
    tok[2, :19] = 0
    cache = text_api.make_cache(cfg, B, T, 8, dtype=bf16, device=_dev())
    from omegalax_b200.models.qwen3.paged_cache import PagedKVCache
    assert isinstance(cache, PagedKVCache)
    logits, cache, _ = text_api.decode(model, cache, tok, 0, cfg)
    seq = tok
    for _ in range(6):
        with torch.no_grad():  # oracle: every sequence on its own, without its padding
            rows = []
            for b in range(B):
                real = seq[b][seq[b] != 0][None]
                hidden, _ = text_api.forward(model, real, 0, cfg)
                rows.append(model.lm_head(hidden[:, -1]))
            full = torch.cat(rows, 0)
        assert _rel_err(logits, full) < 5e-2
        nxt = full[:, 1:].argmax(-1, keepdim=True) + 1
        seq = torch.cat([seq, nxt], dim=1)
        logits, cache, _ = text_api.decode(model, cache, nxt, 0, cfg)
    _check(lib)
    mesh_lib.set_default_mesh(None)


def test_causal_conv1d_silu():
    from omegalax_b200.ops import functional as Fn, reference as R, lib
    torch.manual_seed(11)
    B, T, C = 2, 100, 64
    x = torch.randn(B, T, C, device=_dev()).to(bf16).requires_grad_(True)
    w = (torch.randn(C, 4, device=_dev()) * 0.5).to(bf16).requires_grad_(True)
    y = Fn.causal_conv1d_silu(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    _check(lib)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = R.causal_conv1d(xr.transpose(1, 2), wr, activation_silu=True).transpose(1, 2)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 2e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2


@pytest.mark.parametrize("U,Hk,H,T,with_state", [(128, 2, 4, 200, False), (64, 1, 2, 128, True)])
def test_gated_delta_rule_fwd_bwd(U, Hk, H, T, with_state):
    from omegalax_b200.ops import functional as Fn, reference as R, lib
    torch.manual_seed(5)
    B, A = 2, 128
    dev = _dev()
    q = torch.randn(B, T, Hk, A, device=dev, requires_grad=True)
    k = torch.randn(B, T, Hk, A, device=dev, requires_grad=True)
    v = torch.randn(B, T, H, U, device=dev, requires_grad=True)
    g = (-torch.rand(B, T, H, device=dev) * 0.3).requires_grad_(True)
    beta = torch.sigmoid(torch.randn(B, T, H, device=dev)).requires_grad_(True)
    s0 = (torch.randn(B, H, A, U, device=dev) * 0.1).requires_grad_(True) if with_state else None
    out = Fn.gated_delta_rule(q, k, v, g, beta, initial_state=s0, output_final_state=with_state)
    o, sf = out if with_state else (out, None)
    do = torch.randn_like(o)
    dsf = torch.randn_like(sf) * 0.1 if with_state else None
    loss = (o * do).sum() + ((sf * dsf).sum() if with_state else 0.0)
    loss.backward()
    _check(lib)
    leaves = [q, k, v, g, beta] + ([s0] if with_state else [])
    got = [t.grad.clone() for t in leaves]
    for t in leaves:
        t.grad = None
    rep = H // Hk
    ref = R.chunk_gated_delta_rule(q.repeat_interleave(rep, 2), k.repeat_interleave(rep, 2), v, g, beta,
                                   initial_state=s0, output_final_state=with_state)
    ro, rsf = ref if with_state else (ref, None)
    rl = (ro * do).sum() + ((rsf * dsf).sum() if with_state else 0.0)
    rl.backward()
    assert _rel_err(o, ro) < 1e-4
    if with_state:
        assert _rel_err(sf, rsf) < 1e-4
    for name, a, t in zip(["q", "k", "v", "g", "beta", "s0"], got, leaves):
        assert _rel_err(a, t.grad) < 2e-3, name


def test_gated_rmsnorm_and_layernorm():
    from omegalax_b200.ops import functional as Fn, reference as R, lib
    torch.manual_seed(3)
    dev = _dev()
    M, D = 1000, 128
    x = torch.randn(M, D, device=dev).to(bf16).requires_grad_(True)
    z = torch.randn(M, D, device=dev).to(bf16).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(D, device=dev)).to(bf16).requires_grad_(True)
    y = Fn.rmsnorm_gated(x, w, z, 1e-6)
    dy = torch.randn_like(y)
    y.backward(dy)
    _check(lib)
    xr, zr, wr = (t.detach().float().requires_grad_(True) for t in (x, z, w))
    yr = R.rmsnorm_gated(xr, wr, zr, 1e-6)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 2e-2
    for a, b in ((x.grad, xr.grad), (z.grad, zr.grad), (w.grad, wr.grad)):
        assert _rel_err(a, b) < 3e-2
    for D in (1024, 1152):
        x = torch.randn(300, D, device=dev).to(bf16).requires_grad_(True)
        w = (1 + 0.1 * torch.randn(D, device=dev)).to(bf16).requires_grad_(True)
        b = (0.1 * torch.randn(D, device=dev)).to(bf16).requires_grad_(True)
        y = Fn.layernorm(x, w, b, 1e-6)
        dy = torch.randn_like(y)
        y.backward(dy)
        _check(lib)
        xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
        yr = R.layernorm(xr, wr, br, 1e-6)
        yr.backward(dy.float())
        assert _rel_err(y, yr) < 2e-2
        for a, c in ((x.grad, xr.grad), (w.grad, wr.grad), (b.grad, br.grad)):
            assert _rel_err(a, c) < 3e-2


@pytest.mark.parametrize("E,k,renorm", [(128, 8, True), (512, 10, True), (64, 4, False)])
def test_router_kernel(E, k, renorm):
    from omegalax_b200.ops import moe as moe_ops, lib
    torch.manual_seed(9)
    dev = _dev()
    M = 777
    logits = (torch.randn(M, E, device=dev) * 2).to(bf16).requires_grad_(True)
    probs, w, idx = moe_ops.route(logits, k, renorm)
    gp = torch.randn_like(probs) * 0.1
    gw = torch.randn_like(w)
    (probs * gp).sum().add((w * gw).sum()).backward()
    _check(lib)
    lr = logits.detach().float().requires_grad_(True)
    pr = torch.softmax(lr, -1)
    _, ir = torch.topk(pr, k, dim=-1)
    wr = pr.gather(-1, idx)          # same pick order as the kernel (bf16 logits produce exact ties)
    if renorm:
        wr = wr / wr.sum(-1, keepdim=True).clamp_min(1e-9)
    (pr * gp).sum().add((wr * gw).sum()).backward()
    tie_free = (torch.sort(idx, -1).values == torch.sort(ir, -1).values).all(-1)
    assert tie_free.float().mean() > 0.98
    assert _rel_err(probs, pr) < 1e-5
    assert _rel_err(w, wr) < 1e-5
    assert _rel_err(logits.grad, lr.grad) < 2e-2


def test_moe_mlp_kernel_path_matches_dense_loop():
    from omegalax_b200.ops import moe as moe_ops, lib
    torch.manual_seed(21)
    dev = _dev()
    M, D, F_, E, k = 300, 128, 64, 8, 2
    x = torch.randn(M, D, device=dev).to(bf16).requires_grad_(True)
    wg = (torch.randn(E, 2 * F_, D, device=dev) * D ** -0.5).to(bf16).requires_grad_(True)
    wd = (torch.randn(E, D, F_, device=dev) * F_ ** -0.5).to(bf16).requires_grad_(True)
    logits = torch.randn(M, E, device=dev)
    wts, idx = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    wts = wts.clone().requires_grad_(True)
    y = moe_ops.moe_mlp(x, wts, idx, wg, wd)
    dy = torch.randn_like(y)
    y.backward(dy)
    _check(lib)
    xr, wgr, wdr, wtr = (t.detach().float().requires_grad_(True) for t in (x, wg, wd, wts))
    out = torch.zeros(M, D, device=dev)
    for e in range(E):
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        gu = xr[tok] @ wgr[e].t()
        g, u = gu.chunk(2, -1)
        ye = (torch.nn.functional.silu(g) * u) @ wdr[e].t()
        out = out.index_add(0, tok, ye * wtr[tok, slot].unsqueeze(-1))
    out.backward(dy.float())
    assert _rel_err(y, out) < 3e-2
    assert _rel_err(x.grad, xr.grad) < 4e-2
    assert _rel_err(wts.grad, wtr.grad) < 4e-2
    assert _rel_err(wg.grad, wgr.grad) < 4e-2
    assert _rel_err(wd.grad, wdr.grad) < 4e-2


@pytest.mark.parametrize("rows,other_rows", [(256, None), (1024, 2048), (384, None), (640, 2048)])
@pytest.mark.parametrize("side", [1, 2])
def test_gemm_with_in_kernel_all_gather(side, rows, other_rows, monkeypatch):
    """Gather mode on one GPU: the 'ranks' are four buffers of this GPU, so the copy CTAs, the
    per-chunk counters and the chunk-ordered tile walk are exercised without a second device."""
    from omegalax_b200.ops import kernels as K, lib
    torch.manual_seed(17)
    dev = _dev()
    monkeypatch.setattr(K, "_PAIR_AG", True)   # exercise the CTA-pair kernel's gather mode where the shape allows
    W, Kd, rank = 4, 512, 1        # rows 1024 x 2048 other rows: enough tiles for the CTA-pair kernel
    flags = torch.zeros(W, dtype=torch.int32, device=dev)
    for call in range(2):
        chunks = [torch.randn(rows, Kd, device=dev).to(bf16) for _ in range(W)]
        full = torch.zeros(rows * W, Kd, dtype=bf16, device=dev)
        other = torch.randn(other_rows or (384 if side == 1 else 300), Kd, device=dev).to(bf16)
        y = K.gemm_ag(other, full, [c.data_ptr() for c in chunks], side=side, rank=rank, rows_per_rank=rows,
                      flags=flags, target=8 * (call + 1), copy_ctas=8)
        torch.cuda.synchronize()
        _check(lib)
        want_full = torch.cat(chunks)
        assert torch.equal(full, want_full)
        ref = want_full.float() @ other.float().t() if side == 1 else other.float() @ want_full.float().t()
        assert _rel_err(y, ref) < 1e-2
        assert flags.tolist() == [8 * (call + 1)] * W


def test_gated_delta_rule_strong_decay_against_fp64_recurrence():
    """Decay rates as large as a freshly initialised model produces (|g| up to ~20 per token).
    Ground truth is the token-by-token recurrence in float64; the kernel must be about as close
    to it as the fp32 chunked PyTorch definition is."""
    from omegalax_b200.ops import functional as Fn, reference as R, lib
    torch.manual_seed(13)
    dev = _dev()
    B, T, Hk, H, A, U = 1, 128, 1, 2, 128, 64

    def leaves(dtype):
        torch.manual_seed(13)
        q = torch.randn(B, T, Hk, A, device=dev)
        k = torch.randn(B, T, Hk, A, device=dev)
        v = torch.randn(B, T, H, U, device=dev)
        g = -torch.rand(B, T, H, device=dev) * 20.0
        g[:, ::3] *= 0.01                      # a mix of nearly no decay and very strong decay
        beta = torch.sigmoid(torch.randn(B, T, H, device=dev))
        return [t.to(dtype).requires_grad_(True) for t in (q, k, v, g, beta)]

    do = torch.randn(B, T, H, U, device=dev)
    # float64 recurrence
    q, k, v, g, beta = leaves(torch.float64)
    qn = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * A ** -0.5
    kn = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    qn, kn = qn.repeat_interleave(H // Hk, 2), kn.repeat_interleave(H // Hk, 2)
    S = torch.zeros(B, H, A, U, dtype=torch.float64, device=dev)
    outs = []
    for t in range(T):
        S = S * torch.exp(g[:, t])[..., None, None]
        kv = torch.einsum("bha,bhau->bhu", kn[:, t], S)
        delta = (v[:, t] - kv) * beta[:, t][..., None]
        S = S + torch.einsum("bha,bhu->bhau", kn[:, t], delta)
        outs.append(torch.einsum("bha,bhau->bhu", qn[:, t], S))
    o64 = torch.stack(outs, 1)
    (o64 * do.double()).sum().backward()
    truth = [o64.detach()] + [t.grad.clone() for t in (q, k, v, g, beta)]

    def run(fn):
        ls = leaves(torch.float32)
        o = fn(*ls)
        (o * do).sum().backward()
        return [o.detach()] + [t.grad.clone() for t in ls]

    kern = run(lambda q, k, v, g, b: Fn.gated_delta_rule(q, k, v, g, b))
    _check(lib)
    ref = run(lambda q, k, v, g, b: R.chunk_gated_delta_rule(q.repeat_interleave(H // Hk, 2),
                                                             k.repeat_interleave(H // Hk, 2), v, g, b))
    for name, t64, tk, tr in zip(["o", "dq", "dk", "dv", "dg", "dbeta"], truth, kern, ref):
        ek = float((tk.double() - t64).norm() / (t64.norm() + 1e-30))
        er = float((tr.double() - t64).norm() / (t64.norm() + 1e-30))
        assert ek < max(5e-4, 5 * er), (name, ek, er)


def test_gather_scatter_gelu_kernels():
    from omegalax_b200.ops import functional as Fn, reference as R, lib
    torch.manual_seed(2)
    dev = _dev()
    M, D, n = 500, 256, 77
    x = torch.randn(M, D, device=dev).to(bf16).requires_grad_(True)
    src = torch.randn(n, D, device=dev).to(bf16).requires_grad_(True)
    pos = torch.randperm(M, device=dev)[:n].sort().values
    for replace in (False, True):
        y = Fn.scatter_rows(x, pos, src, replace=replace)
        dy = torch.randn_like(y)
        y.backward(dy)
        xr, sr = x.detach().float().requires_grad_(True), src.detach().float().requires_grad_(True)
        base = xr
        if replace:
            keep = torch.ones(M, 1, device=dev).index_fill(0, pos, 0.0)
            base = xr * keep
        yr = base.index_add(0, pos, sr)
        yr.backward(dy.float())
        assert _rel_err(y, yr) < 1e-2
        assert _rel_err(x.grad, xr.grad) < 1e-2 and _rel_err(src.grad, sr.grad) < 1e-2
        x.grad = None
        src.grad = None
    table = torch.randn(48 * 48, D, device=dev).to(bf16).requires_grad_(True)
    N = 300
    idx = torch.randint(0, 48 * 48, (N, 4), device=dev)
    w = torch.rand(N, 4, device=dev)
    o = Fn.gather4(table, idx, w)
    do = torch.randn_like(o)
    o.backward(do)
    tr = table.detach().float().requires_grad_(True)
    orf = (tr[idx.reshape(-1)].view(N, 4, D) * w.unsqueeze(-1)).sum(1)
    orf.backward(do.float())
    assert _rel_err(o, orf) < 1e-2 and _rel_err(table.grad, tr.grad) < 2e-2
    z = (torch.randn(1000, 64, device=dev) * 2).to(bf16).requires_grad_(True)
    g = Fn.gelu_tanh(z)
    dg = torch.randn_like(g)
    g.backward(dg)
    zr = z.detach().float().requires_grad_(True)
    gr = R.gelu_tanh(zr)
    gr.backward(dg.float())
    assert _rel_err(g, gr) < 1e-2 and _rel_err(z.grad, zr.grad) < 2e-2
    _check(lib)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("lens", [[512], [200, 456, 77], [128, 1]])
def test_attention_head_dim_256_forward_backward(causal, lens):
    """256-wide heads (Qwen3.5 gated attention, 16 query heads per kv head): forward (two warpgroups
    share the output by head-dim halves) and backward (one pass per head-dim half) on packed
    sequences of uneven length, per element against fp32 PyTorch."""
    from omegalax_b200.ops import functional as Fn, reference as R, lib
    torch.manual_seed(17)
    dev = _dev()
    H, G, HD = 4, 2, 256
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=dev, dtype=torch.int32)
    N = sum(lens)
    q = torch.randn(N, H, HD, device=dev).to(bf16).requires_grad_(True)
    k = torch.randn(N, G, HD, device=dev).to(bf16).requires_grad_(True)
    v = torch.randn(N, G, HD, device=dev).to(bf16).requires_grad_(True)
    o = Fn.flash_attention(q, k, v, cu, max(lens), scale=HD ** -0.5, causal=causal)
    do = torch.randn_like(o)
    o.backward(do)
    _check(lib)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = R.attention_varlen(qr, kr, vr, cu, causal=causal, scale=HD ** -0.5)
    ref.backward(do.float())
    torch.testing.assert_close(o.float(), ref, rtol=2.0 ** -6, atol=2e-2)
    for got, want in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        torch.testing.assert_close(got.float(), want, rtol=2.0 ** -5, atol=3e-2 * float(want.abs().max()))


def test_sigmoid_gate_on_a_strided_gate_view():
    from omegalax_b200.ops import functional as Fn, lib
    torch.manual_seed(19)
    M, H, Kd = 300, 4, 256
    fused = torch.randn(M, H * 2 * Kd + 64, device=_dev()).to(bf16).requires_grad_(True)   # [q | gate] per head, then more
    o = torch.randn(M, H, Kd, device=_dev()).to(bf16).requires_grad_(True)
    gate = fused[:, : H * 2 * Kd].view(M, H, 2, Kd)[:, :, 1]
    y = Fn.sigmoid_gate(o, gate)
    dy = torch.randn_like(y)
    y.backward(dy)
    _check(lib)
    fr, orf = fused.detach().float().requires_grad_(True), o.detach().float().requires_grad_(True)
    yr = orf * torch.sigmoid(fr[:, : H * 2 * Kd].view(M, H, 2, Kd)[:, :, 1])
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, rtol=2.0 ** -7, atol=1e-2)
    torch.testing.assert_close(o.grad.float(), orf.grad, rtol=2.0 ** -6, atol=1e-2)
    torch.testing.assert_close(fused.grad.float(), fr.grad, rtol=2.0 ** -6, atol=1e-2)


def test_attention_backward_head_dim_64_varlen():
    """64-wide heads (vision tower): non-causal packed sequences of different lengths."""
    from omegalax_b200.ops import functional as Fn, reference as R, lib
    torch.manual_seed(12)
    dev = _dev()
    H, HD = 4, 64
    lens = [200, 64, 333]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=dev, dtype=torch.int32)
    N = sum(lens)
    q, k, v = (torch.randn(N, H, HD, device=dev).to(bf16).requires_grad_(True) for _ in range(3))
    o = Fn.flash_attention(q, k, v, cu, max(lens), scale=HD ** -0.5, causal=False)
    do = torch.randn_like(o)
    o.backward(do)
    _check(lib)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = R.attention_varlen(qr, kr, vr, cu, causal=False, scale=HD ** -0.5)
    ref.backward(do.float())
    assert _rel_err(o, ref) < 2e-2
    for a, b in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert _rel_err(a, b) < 3e-2


@pytest.mark.parametrize("M,N,K", [(512, 512, 256), (1000, 768, 384), (4096, 1536, 2048), (256, 256, 64)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_cta_pair_layouts(M, N, K, a_mn, b_mn):
    from omegalax_b200.ops import kernels as Kn, lib
    torch.manual_seed(1)
    a = torch.randn((K, M) if a_mn else (M, K), device=_dev()).to(bf16)
    b = torch.randn((K, N) if b_mn else (N, K), device=_dev()).to(bf16)
    c = Kn.gemm(a, b, a_mn=a_mn, b_mn=b_mn, pair=True)
    torch.cuda.synchronize()
    _check(lib)
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    assert _rel_err(c, af @ bf) < 1e-2


def test_gemm_cta_pair_epilogues():
    from omegalax_b200.ops import kernels as Kn, lib
    torch.manual_seed(2)
    M, N, K = 1024, 1024, 512
    a = torch.randn(M, K, device=_dev()).to(bf16)
    b = torch.randn(N, K, device=_dev()).to(bf16)
    res = torch.randn(M, N, device=_dev()).to(bf16)
    ref = a.float() @ b.float().t()
    c = Kn.gemm(a, b, residual=res, pair=True)
    assert _rel_err(c, ref + res.float()) < 1e-2
    acc = torch.ones(M, N, device=_dev())
    Kn.gemm(a, b, out=acc, accumulate=True, pair=True)
    assert _rel_err(acc, ref + 1.0) < 1e-2
    _check(lib)


_DEBUG_SCRIPT = r"""
import torch
from omegalax_b200.ops import kernels as K, lib
assert lib.debug_enabled() and str(lib.LIB_PATH).endswith("_debug.so")
dev = torch.device("cuda", 0)
table = torch.randn(64, 32, device=dev).to(torch.bfloat16)
try:
    K.embedding_fwd(torch.tensor([1, 64], device=dev), table)
    raise SystemExit("bad id was not caught")
except IndexError as e:
    assert "value 64 at flat position 1" in str(e), e
a = torch.randn(300, 136, device=dev).to(torch.bfloat16)
b = torch.randn(520, 136, device=dev).to(torch.bfloat16)
for pair in (False, True):
    out = K.gemm(a, b, pair=pair)
    torch.testing.assert_close(out.float(), a.float() @ b.float().t(), rtol=2 ** -7, atol=0.1)
N, H, G, Kd = 256, 2, 1, 128
q = torch.randn(N, H, Kd, device=dev).to(torch.bfloat16)
k = torch.randn(N, G, Kd, device=dev).to(torch.bfloat16)
v = torch.randn(N, G, Kd, device=dev).to(torch.bfloat16)
cu = torch.tensor([0, N], device=dev, dtype=torch.int32)
o, lse = K.attn_fwd(q, k, v, cu, N, Kd ** -0.5, True)
K.attn_bwd(q, k, v, o, lse, torch.randn_like(o), cu, N, Kd ** -0.5, True)
torch.cuda.synchronize()
lib.check_status()          # guard bands around the attention scratch intact, no store outside an output
print("debug ok")
"""


def test_debug_mode_catches_bad_indices_on_the_host_and_keeps_kernels_correct():
    """OMEGALAX_B200_DEBUG=1 in a fresh process: the debug library is built and loaded, an
    out-of-range token id raises on the host before any launch, kernels still agree with PyTorch
    and the scratch guard bands stay intact."""
    import os
    import subprocess
    import sys

    env = dict(os.environ, OMEGALAX_B200_DEBUG="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", _DEBUG_SCRIPT], env=env, cwd=root, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0 and "debug ok" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
