// NVLink peer-memory substrate: allocation + CUDA IPC handle exchange helpers, a bounded
// device-side barrier over peer flags, and the pull all-gather used by the sharded engine.
//
// Every GPU allocates the same buffers ("symmetric heap"); handles are exchanged once through
// the host process group and each rank maps all peers' buffers.  Kernels then read and write
// peer memory with ordinary ld/st/red instructions over NVLink; nothing here uses cluster
// multicast loads.  All waits on peer flags are bounded and report through the status word.
#include "host_utils.h"
#include "sm100_common.cuh"

namespace ob {

constexpr int kMaxRanks = 8;

struct PeerPtrs {
  void* p[kMaxRanks];
};

// ---------------------------------------------------------------- barrier
// flags layout on every rank: uint32 slots[kMaxRanks]; rank r writes its epoch into slot r of
// every peer, then waits until all slots of its own array have reached the epoch.
__global__ void symm_barrier_kernel(PeerPtrs flags, int world, int rank, uint32_t epoch,
                                    long long budget_cycles, int* status) {
  const int t = threadIdx.x;
  if (t < world) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(flags.p[t]) + rank;
    __threadfence_system();
    st_release_sys(dst, epoch);
  }
  if (t < world) {
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[rank]) + t;
    flag_wait_ge<true>(mine, epoch, budget_cycles, status, OB_ERR_WAIT_FLAG);
  }
}

// ---------------------------------------------------------------- pull all-gather
// Copy segments: for segment s, `elems16` 16-byte units from peer `src_rank` at byte offset
// `src_off` (inside that peer's shard buffer) to the local buffer at `dst_off`.
struct CopySeg {
  long long src_off, dst_off, bytes;
  int src_rank, pad;
};

__global__ void allgather_pull_kernel(PeerPtrs shard, uint8_t* __restrict__ dst,
                                      const CopySeg* __restrict__ segs, int nsegs) {
  // grid.y walks segments, grid.x * blockDim.x threads stride over the 16-byte units of one
  for (int s = blockIdx.y; s < nsegs; s += gridDim.y) {
    const CopySeg sg = segs[s];
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(shard.p[sg.src_rank]) + sg.src_off);
    uint4* d = reinterpret_cast<uint4*>(dst + sg.dst_off);
    const long long n = sg.bytes >> 4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    // four independent 16-byte loads in flight per thread to cover the NVLink latency
    for (; i + 3 * stride < n; i += 4 * stride) {
      uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], e = src[i + 3 * stride];
      d[i] = a; d[i + stride] = b; d[i + 2 * stride] = c; d[i + 3 * stride] = e;
    }
    for (; i < n; i += stride) d[i] = src[i];
  }
}

// ---------------------------------------------------------------- pull reduce-scatter
// out[i] += sum over ranks r != self of peer_full[r][my_off + i]  (fp32); used for parameters
// whose gradient cannot go through the GEMM peer-reduce epilogue (norm weights, embeddings).
__global__ void reduce_scatter_pull_kernel(PeerPtrs full, float* __restrict__ out, long long src_off_elems,
                                           long long n, int world, int rank, int include_self) {
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = reinterpret_cast<float4*>(out)[i];
    for (int r = 0; r < world; ++r) {
      if (r == rank && !include_self) continue;
      float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(full.p[r]) + src_off_elems)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(out)[i] = acc;
  }
  if (blockIdx.x == 0) {
    for (long long i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x) {
      float a = out[i];
      for (int r = 0; r < world; ++r) {
        if (r == rank && !include_self) continue;
        a += (reinterpret_cast<const float*>(full.p[r]) + src_off_elems)[i];
      }
      out[i] = a;
    }
  }
}

// ---------------------------------------------------------------- scatter-add of small gradients
// Gradients of the parameters that do not go through a GEMM epilogue (norm weights, biases, router
// tables): every rank holds a full fp32 gradient of the unit's parameters and adds each element
// into the owning rank's gradient shard with an fp32 reduction over NVLink (into every rank's copy
// for replicated parameters), then clears its local buffer.  No rank waits for another here: the
// reductions are ordered by the same end-of-backward barrier as the weight-gradient epilogues, so
// a layer's backward has no cross-rank synchronisation point at all.
struct ScatSeg {
  long long src_off, dst_off;   // elements: into the local full buffer / into every rank's shard buffer
  int numel, shard_numel;       // shard_numel == numel for replicated parameters
  int sharded, pad;
};

__global__ void peer_scatter_add_kernel(float* __restrict__ src, PeerPtrs dst, const ScatSeg* __restrict__ segs,
                                        int nsegs, int world) {
  for (int s = blockIdx.y; s < nsegs; s += gridDim.y) {
    const ScatSeg sg = segs[s];
    float* sp = src + sg.src_off;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < sg.numel; i += gridDim.x * blockDim.x) {
      const float v = sp[i];
      sp[i] = 0.f;
      if (v == 0.f) continue;
      if (sg.sharded) {
        const int owner = i / sg.shard_numel;
        atomicAdd(reinterpret_cast<float*>(dst.p[owner]) + sg.dst_off + (i - owner * sg.shard_numel), v);
      } else {
        for (int r = 0; r < world; ++r) atomicAdd(reinterpret_cast<float*>(dst.p[r]) + sg.dst_off + i, v);
      }
    }
  }
}

// ---------------------------------------------------------------- slab sum (two-phase reduce-scatter)
// out[i] = sum over the `slots` slabs of staging[s * slab_elems + i] (+ residual[i]); bf16 in and out,
// fp32 accumulation.  Second phase of the GEMM -> reduce-scatter whose first phase stored every
// sender's partial tile into its own slab of this GPU's staging buffer.
__global__ void slab_sum_kernel(const bf16* __restrict__ staging, int slots, long long slab_elems,
                                const bf16* __restrict__ residual, bf16* __restrict__ out) {
  const long long nv = slab_elems >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (residual) {
      const uint4 q = reinterpret_cast<const uint4*>(residual)[i];
      const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(u[j]);
        acc[2 * j] = f.x; acc[2 * j + 1] = f.y;
      }
    }
    for (int s = 0; s < slots; ++s) {
      const uint4 q = reinterpret_cast<const uint4*>(staging + (long long)s * slab_elems)[i];
      const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(u[j]);
        acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

}  // namespace ob

using namespace ob;

extern "C" {

int ob_peer_scatter_add(float* src, void* const* dst_ptrs, int world, const void* segs, int nsegs, int max_numel,
                        cudaStream_t stream) {
  if (world > kMaxRanks) return 6003;
  if (nsegs <= 0) return 0;
  PeerPtrs d = {};
  for (int i = 0; i < world; ++i) d.p[i] = dst_ptrs[i];
  int bx = (max_numel + 255) / 256;
  if (bx > 64) bx = 64;
  if (bx < 1) bx = 1;
  dim3 grid(bx, nsegs < 64 ? nsegs : 64);
  peer_scatter_add_kernel<<<grid, 256, 0, stream>>>(src, d, (const ScatSeg*)segs, nsegs, world);
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_slab_sum(const void* staging, int slots, long long slab_elems, const void* residual, void* out,
                cudaStream_t stream) {
  if (slab_elems <= 0) return 0;
  if (slab_elems % 8) return 6001;
  if (((uintptr_t)staging | (uintptr_t)out | (uintptr_t)residual) & 15) return 6002;
  long long blocks = (slab_elems / 8 + 255) / 256;
  const long long cap = (long long)num_sms() * 8;
  slab_sum_kernel<<<(unsigned)(blocks > cap ? cap : blocks), 256, 0, stream>>>((const bf16*)staging, slots, slab_elems,
                                                                             (const bf16*)residual, (bf16*)out);
  OB_CHECK_LAUNCH();
  return 0;
}

// ---- allocation / IPC (host side)
int ob_symm_alloc(void** out, long long bytes) {
  cudaError_t e = cudaMalloc(out, (size_t)bytes);
  if (e != cudaSuccess) return 1000 + (int)e;
  e = cudaMemset(*out, 0, (size_t)bytes);
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
int ob_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : 1; }
int ob_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return 1000 + (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
int ob_ipc_open_handle(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
int ob_ipc_close_handle(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : 1; }
int ob_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }

// ---- device barrier over peer flags (bounded wait of ~budget_ms)
int ob_symm_barrier(void* const* flag_ptrs, int world, int rank, unsigned epoch, int budget_ms, int* status,
                    cudaStream_t stream) {
  if (world > kMaxRanks) return 6003;
  PeerPtrs f = {};
  for (int i = 0; i < world; ++i) f.p[i] = flag_ptrs[i];
  long long cycles = (long long)budget_ms * 2000000ll;
  symm_barrier_kernel<<<1, 32, 0, stream>>>(f, world, rank, epoch, cycles, status);
  OB_CHECK_LAUNCH();
  return 0;
}

// ---- pull all-gather: segs is a device array of CopySeg (4 x int64 words each)
int ob_allgather_pull(void* const* shard_ptrs, int world, void* dst, const void* segs, int nsegs,
                      cudaStream_t stream) {
  if (world > kMaxRanks) return 6003;
  if (nsegs <= 0) return 0;
  PeerPtrs s = {};
  for (int i = 0; i < world; ++i) s.p[i] = shard_ptrs[i];
  dim3 grid(num_sms() * 2 / (nsegs < 8 ? nsegs : 8) + 1, nsegs < 8 ? nsegs : 8);
  allgather_pull_kernel<<<grid, 256, 0, stream>>>(s, (uint8_t*)dst, (const CopySeg*)segs, nsegs);
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_reduce_scatter_pull(void* const* full_ptrs, int world, int rank, float* out, long long src_off_elems,
                           long long n, int include_self, cudaStream_t stream) {
  if (world > kMaxRanks) return 6003;
  if (n <= 0) return 0;
  PeerPtrs f = {};
  for (int i = 0; i < world; ++i) f.p[i] = full_ptrs[i];
  long long blocks = (n / 4 + 255) / 256;
  long long cap = (long long)num_sms() * 4;
  reduce_scatter_pull_kernel<<<(unsigned)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks)), 256, 0, stream>>>(
      f, out, src_off_elems, n, world, rank, include_self);
  OB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Expert-parallel token exchange over peer memory (dispatch / combine).
//
// push: for every (token, slot) pair p, the token's row is written into the receive buffer of
//       the GPU that owns the chosen expert, at the row the routing plan assigned to it (the
//       router permutation is folded into the destination address).  An optional per-pair
//       scale implements the backward of the weighted combine.
// pull: every token gathers its k expert outputs from the owners' buffers and forms the
//       weighted sum in fp32 (weighted un-permute); optionally also the per-pair dot product
//       with an upstream gradient (gradient of the routing weights).
// One warp per pair (push) or per token (pull); rows are moved as 16-byte vectors.
namespace ob {

// Every rank writes its per-expert pair counts into row `rank` of every peer's count table
// (W x E ints on each GPU): after the next device barrier all ranks hold the same table and derive
// the same routing plan from it, without a host-launched collective.
__global__ void ep_publish_counts_kernel(PeerPtrs tbl, const int* __restrict__ mine, int E, int world, int rank) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= world * E) return;
  const int peer = t / E, e = t - peer * E;
  reinterpret_cast<int*>(tbl.p[peer])[rank * E + e] = mine[e];
}

__global__ void ep_push_kernel(PeerPtrs dst, const bf16* __restrict__ src, const int* __restrict__ src_row,
                               const int* __restrict__ dst_rank, const int* __restrict__ dst_row,
                               const float* __restrict__ scale, long long P, int D) {
  const long long p = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (p >= P) return;
  if (dst_row[p] < 0) return;   // dropped pair (receive buffer overflow)
  const uint4* s = reinterpret_cast<const uint4*>(src + (long long)src_row[p] * D);
  uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst.p[dst_rank[p]]) + (long long)dst_row[p] * D);
  const int nv = D >> 3;
  if (scale == nullptr) {
    for (int i = lane; i < nv; i += 32) d[i] = s[i];
  } else {
    const float sc = scale[p];
    for (int i = lane; i < nv; i += 32) {
      uint4 q = s[i];
      uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16(u[j]);
        u[j] = pack_bf16(f.x * sc, f.y * sc);
      }
      d[i] = make_uint4(u[0], u[1], u[2], u[3]);
    }
  }
}

__global__ void ep_pull_kernel(PeerPtrs src, bf16* __restrict__ out, const int* __restrict__ src_rank,
                               const int* __restrict__ src_row, const float* __restrict__ w,
                               const bf16* __restrict__ g, float* __restrict__ dot_out, long long M, int k, int D) {
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= M) return;
  const int nv = D >> 3;
  for (int c0 = 0; c0 < nv; c0 += 32) {
    const int i = c0 + lane;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float gv[8];
    if (g != nullptr && i < nv) {
      uint4 q = reinterpret_cast<const uint4*>(g + t * D)[i];
      uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16(u[j]);
        gv[2 * j] = f.x; gv[2 * j + 1] = f.y;
      }
    }
    for (int j = 0; j < k; ++j) {
      const long long p = t * k + j;
      float dot = 0.f;
      if (i < nv && src_row[p] >= 0) {
        const uint4 q = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(src.p[src_rank[p]]) +
                                                       (long long)src_row[p] * D)[i];
        const float wj = w ? w[p] : 1.f;
        uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f = unpack_bf16(u[e]);
          acc[2 * e] += wj * f.x;
          acc[2 * e + 1] += wj * f.y;
          if (g != nullptr) dot += gv[2 * e] * f.x + gv[2 * e + 1] * f.y;
        }
      }
      if (g != nullptr) {
        dot = warp_sum(dot);
        if (lane == 0) {
          if (c0 == 0) dot_out[p] = dot; else dot_out[p] += dot;
        }
      }
    }
    if (out != nullptr && i < nv) {
      uint4 o;
      o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
      o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out + t * D)[i] = o;
    }
  }
}

}  // namespace ob

extern "C" {

int ob_ep_publish_counts(void* const* tbl_ptrs, int world, int rank, const int* mine, int E, cudaStream_t stream) {
  if (world > kMaxRanks) return 6003;
  if (E <= 0) return 0;
  PeerPtrs t = {};
  for (int i = 0; i < world; ++i) t.p[i] = tbl_ptrs[i];
  const int n = world * E;
  ep_publish_counts_kernel<<<(n + 255) / 256, 256, 0, stream>>>(t, mine, E, world, rank);
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_ep_push(void* const* dst_ptrs, int world, const void* src, const int* src_row, const int* dst_rank,
               const int* dst_row, const float* scale, long long P, int D, cudaStream_t stream) {
  if (world > kMaxRanks) return 6003;
  if (D % 8) return 6001;
  if (P <= 0) return 0;
  PeerPtrs d = {};
  for (int i = 0; i < world; ++i) d.p[i] = dst_ptrs[i];
  long long blocks = (P * 32 + 255) / 256;
  ep_push_kernel<<<(unsigned)blocks, 256, 0, stream>>>(d, (const bf16*)src, src_row, dst_rank, dst_row, scale, P, D);
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_ep_pull(void* const* src_ptrs, int world, void* out, const int* src_rank, const int* src_row,
               const float* w, const void* g, float* dot_out, long long M, int k, int D, cudaStream_t stream) {
  if (world > kMaxRanks) return 6003;
  if (D % 8) return 6001;
  if (M <= 0) return 0;
  PeerPtrs s = {};
  for (int i = 0; i < world; ++i) s.p[i] = src_ptrs[i];
  long long blocks = (M * 32 + 255) / 256;
  ep_pull_kernel<<<(unsigned)blocks, 256, 0, stream>>>(s, (bf16*)out, src_rank, src_row, w, (const bf16*)g, dot_out,
                                                       M, k, D);
  OB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
