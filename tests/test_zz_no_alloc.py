"""The allocation-free attention backward (built-in scratch) against the regular entry point.

Some callers of the library cannot allocate device memory -- they run inside a fixed memory
budget, or inside a process whose allocator they do not own -- so ``ob_attn_bwd_noalloc`` keeps
its work buffers in a fixed array of the library image.  This file is collected last on
purpose: the new entry point shares one scratch array per GPU, and every other test should
have run before a failure here stops the session.  It calls the exported C symbol directly,
twice in a row, because the second call sees what the first one left in the scratch.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sig(fn, n_ptr_head):
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    fn.argtypes = [P] * n_ptr_head + [I, I, L, I, I, I, L, L, L, L, L, L, L, F, I, P, P]
    fn.restype = I


def test_noalloc_matches_regular_entry_point_twice():
    from omegalax_b200.ops import kernels as Kn, lib

    L = lib.load()
    fn = L.ob_attn_bwd_noalloc
    _sig(fn, 10)  # q k v out dout lse dq dk dv cu_seqlens
    dev = torch.device("cuda", 0)
    bf16 = torch.bfloat16
    B, T, H, G, HD = 2, 384, 4, 2, 128
    N = B * T
    st = lib.status_tensor(dev)
    for trial in range(2):  # two calls in a row share (and must re-initialise) the scratch
        torch.manual_seed(20 + trial)
        q = torch.randn(N, H, HD, device=dev).to(bf16)
        k = torch.randn(N, G, HD, device=dev).to(bf16)
        v = torch.randn(N, G, HD, device=dev).to(bf16)
        do = torch.randn(N, H, HD, device=dev).to(bf16)
        cu = torch.arange(B + 1, device=dev, dtype=torch.int32) * T
        scale = HD ** -0.5
        o, lse = Kn.attn_fwd(q, k, v, cu, T, scale, True)
        ref_dq, ref_dk, ref_dv = Kn.attn_bwd(q, k, v, o, lse, do, cu, T, scale, True)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(dev)
        # memory_allocated only sees PyTorch's caching allocator; the driver's free-byte count would
        # also move if the entry point called cudaMalloc / cudaFree itself (checked from the second
        # call on: the first call on a device may load the kernel image)
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(), dq.data_ptr(),
                dk.data_ptr(), dv.data_ptr(), cu.data_ptr(), B, T, N, H, G, HD, q.stride(0), k.stride(0), v.stride(0),
                o.stride(0), do.stride(0), dk.stride(0), dv.stride(0), scale, 1, st.data_ptr(),
                torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info(dev)[0]
        lib.check_status()
        assert torch.cuda.memory_allocated(dev) == before
        if trial > 0:
            assert free_after == free_before
        for got, want in ((dq, ref_dq), (dk, ref_dk), (dv, ref_dv)):
            err = float((got.float() - want.float()).abs().max() / (want.float().abs().max() + 1e-6))
            assert err < 3e-2, err
        # and against the fp32 PyTorch definition of the same gradients
        from omegalax_b200.ops import reference as R

        qr, kr, vr = (t.float().view(B, T, -1, HD).requires_grad_(True) for t in (q, k, v))
        R.attention(qr, kr, vr, causal=True, scale=scale).backward(do.float().view(B, T, H, HD))
        for got, want in ((dq, qr.grad.reshape(N, H, HD)), (dk, kr.grad.reshape(N, G, HD)), (dv, vr.grad.reshape(N, G, HD))):
            err = float((got.float() - want).abs().max() / (want.abs().max() + 1e-6))
            assert err < 3e-2, err


def test_noalloc_rejects_other_head_widths():
    from omegalax_b200.ops import lib

    fn = lib.load().ob_attn_bwd_noalloc
    _sig(fn, 10)
    # the built-in scratch is laid out for 128-wide heads: 256 is refused before anything is launched
    rc = fn(None, None, None, None, None, None, None, None, None, None, 1, 128, 128, 2, 1, 256, 512, 256, 256,
            512, 512, 256, 256, 0.1, 1, None, None)
    assert rc == 6005


def test_noalloc_rejects_problems_beyond_its_scratch():
    from omegalax_b200.ops import lib

    L = lib.load()
    fn = L.ob_attn_bwd_noalloc
    _sig(fn, 10)
    # rows * heads = 40000 * 8 > 32768: refused before anything is launched (pointers unused)
    rc = fn(None, None, None, None, None, None, None, None, None, None, 1, 40000, 40000, 8, 2, 128, 1024, 256, 256,
            1024, 1024, 256, 256, 0.1, 1, None, None)
    assert rc == 6100
