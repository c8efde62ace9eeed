// Attention backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for hosts of this
// library that cannot call cudaMalloc themselves or hand us buffers beyond their inputs and
// outputs: code running under a fixed memory budget that was carved up at start-up, plug-ins
// loaded into a process whose allocator they do not own, and real-time loops in which an
// allocation (and the implicit synchronisation it can cause) is not acceptable.
//
// ob_attn_bwd needs two work buffers besides its inputs and outputs: the per-row dot product
// delta[H, rows] and an fp32 accumulator for dQ of shape [rows, H, 128].  Here both live in a
// fixed array inside the library's device image, so the call allocates nothing (no cudaMalloc,
// cudaFree, or allocating library routine).  The price is a size limit and shared state:
//
//   * rows * H must not exceed OB_ATTN_NOALLOC_MAX_ROW_HEADS (32768), i.e. 16 MiB for the dQ
//     accumulator plus 128 KiB for delta.  Larger problems are rejected with code 6100 and
//     nothing is launched.  Every GPU on which the library is loaded holds this array until the
//     process exits, whether or not the entry point is ever called.
//   * All calls on one GPU share the array.  It keeps whatever the previous call left there;
//     the call itself clears the part that must start at zero (the dQ accumulator), so callers
//     need not.  Two calls that may overlap on the GPU (different streams, or concurrent
//     processes cannot share it at all) race on the array: issue them on one stream or order
//     them with events.
//   * The first call on each device looks up the device address of the array (with that device
//     current) and caches it; make that first call outside of any stream capture.
//
// Arguments are those of ob_attn_bwd without the two scratch pointers; head_dim must be 128 (the
// scratch is laid out for that width; other widths return 6005 and launch nothing).  One process
// may call it on several devices: the address cache and the kernel's shared-memory attribute are
// kept per device.  Returns 0 on success, 6100 if the problem exceeds the built-in scratch, 6101 if
// the address lookup failed, otherwise the code of ob_attn_bwd.
#pragma once
#include <cuda_runtime.h>

#define OB_ATTN_NOALLOC_MAX_ROW_HEADS 32768

#ifdef __cplusplus
extern "C" {
#endif

int ob_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out, const void* dout,
                        const float* lse, void* dq, void* dk, void* dv, const int* cu_seqlens, int B,
                        int max_seqlen, long long total_rows, int H, int G, int HD, long long q_row_stride,
                        long long k_row_stride, long long v_row_stride, long long o_row_stride,
                        long long do_row_stride, long long dk_row_stride, long long dv_row_stride, float scale,
                        int causal, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
