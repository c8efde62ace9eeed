// K9: mixture-of-experts routing.  One warp per token evaluates the fp32 softmax over the
// experts, picks the top-k (ties to the lower expert id), renormalises with clip(sum, 1e-9)
// and counts the picks per expert (omegalax/models/qwen3/model.py:75-82 for the arithmetic).
// A single-CTA scan turns the counts into segment offsets padded to multiples of 128 rows and
// a second pass assigns every (token, slot) pair its row in the expert-sorted buffer.  The rows
// themselves are moved by the dispatch / combine kernels of the expert-parallel path.
#include "host_utils.h"
#include "sm100_common.cuh"

namespace ob {

constexpr int kMaxEPL = 16;   // experts per lane: E <= 512
constexpr int kMaxTopK = 16;

__global__ void router_topk_kernel(const bf16* __restrict__ logits, float* __restrict__ probs,
                                   float* __restrict__ weights, int* __restrict__ idx, int* __restrict__ counts,
                                   long long M, int E, int k, int renorm) {
  const int lane = threadIdx.x & 31;
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (row >= M) return;
  const int epl = E >> 5;
  float v[kMaxEPL];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxEPL; ++i) {
    v[i] = -INFINITY;
    if (i < epl) {
      v[i] = __bfloat162float(logits[row * E + lane + 32 * i]);
      mx = fmaxf(mx, v[i]);
    }
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxEPL; ++i)
    if (i < epl) {
      v[i] = expf(v[i] - mx);
      sum += v[i];
    }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int i = 0; i < kMaxEPL; ++i)
    if (i < epl) {
      v[i] *= inv;
      probs[row * E + lane + 32 * i] = v[i];
    }
  float wsel = 0.f;   // lane r keeps the r-th pick
  int isel = 0;
  float tot = 0.f;
  for (int r = 0; r < k; ++r) {
    float best = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxEPL; ++i)
      if (i < epl && v[i] > best) { best = v[i]; bi = lane + 32 * i; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob_ = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob_ > best || (ob_ == best && oi < bi)) { best = ob_; bi = oi; }
    }
    if ((bi & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kMaxEPL; ++i)
        if (i == (bi >> 5)) v[i] = -1.f;   // taken
    }
    if (bi >= E) {  // only with NaN probabilities (no comparison succeeds): keep the ids in range
      bi = r;
      best = 0.f;
    }
    if (lane == r) { wsel = best; isel = bi; }
    tot += best;
  }
  if (lane < k) {
    const float w = renorm ? wsel / fmaxf(tot, 1e-9f) : wsel;
    weights[row * k + lane] = w;
    idx[row * k + lane] = isel;
    if (counts) atomicAdd(counts + isel, 1);
  }
}

// dlogits = probs * (dP - <probs, dP>), dP = dprobs + scatter(d p_selected)
__global__ void router_topk_bwd_kernel(const float* __restrict__ probs, const float* __restrict__ weights,
                                       const int* __restrict__ idx, const float* __restrict__ dweights,
                                       const float* __restrict__ dprobs, bf16* __restrict__ dlogits, long long M,
                                       int E, int k, int renorm) {
  const int lane = threadIdx.x & 31;
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (row >= M) return;
  const int epl = E >> 5;
  float p[kMaxEPL], dP[kMaxEPL];
#pragma unroll
  for (int i = 0; i < kMaxEPL; ++i) {
    p[i] = 0.f; dP[i] = 0.f;
    if (i < epl) {
      p[i] = probs[row * E + lane + 32 * i];
      if (dprobs) dP[i] = dprobs[row * E + lane + 32 * i];
    }
  }
  // selected entries: lane r holds pick r
  float w = 0.f, dw = 0.f;
  int e = -1;
  if (lane < k) { w = weights[row * k + lane]; dw = dweights[row * k + lane]; e = idx[row * k + lane]; }
  float dps = dw;
  if (renorm) {
    float psel = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxEPL; ++i) {
      // fetch p[e] from its owner lane
      const float cand = __shfl_sync(0xffffffffu, p[i], e < 0 ? 0 : (e & 31));
      if (e >= 0 && (e >> 5) == i) psel = cand;
    }
    const float s = fmaxf(warp_sum(lane < k ? psel : 0.f), 1e-9f);
    const float c = warp_sum(lane < k ? dw * w : 0.f);
    dps = (dw - c) / s;
  }
  for (int r = 0; r < k; ++r) {
    const int er = __shfl_sync(0xffffffffu, e, r);
    const float dr = __shfl_sync(0xffffffffu, dps, r);
    if ((er & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kMaxEPL; ++i)
        if (i == (er >> 5)) dP[i] += dr;
    }
  }
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxEPL; ++i) dot = fmaf(p[i], dP[i], dot);
  dot = warp_sum(dot);
#pragma unroll
  for (int i = 0; i < kMaxEPL; ++i)
    if (i < epl) dlogits[row * E + lane + 32 * i] = __float2bfloat16(p[i] * (dP[i] - dot));
}

// counts[E] -> offsets[E+1] (segments padded to multiples of `pad`), cursors zeroed.  One CTA.
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ cursor,
                                   int E, int pad) {
  __shared__ int sh[1024];
  const int t = threadIdx.x;
  int c = 0;
  if (t < E) c = (counts[t] + pad - 1) / pad * pad;
  sh[t] = c;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const int add = (t >= o) ? sh[t - o] : 0;
    __syncthreads();
    sh[t] += add;
    __syncthreads();
  }
  if (t < E) {
    offsets[t + 1] = sh[t];
    cursor[t] = 0;
  }
  if (t == 0) offsets[0] = 0;
}

__global__ void moe_count_kernel(const int* __restrict__ idx, int* __restrict__ counts, long long P, int E) {
  const long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (p >= P) return;
  const int e = idx[p];
  if (e >= 0 && e < E) atomicAdd(counts + e, 1);   // ids out of range are ignored, never dereferenced
}

__global__ void moe_dest_kernel(const int* __restrict__ idx, const int* __restrict__ offsets, int* __restrict__ cursor,
                                int* __restrict__ dest, long long P, int E) {
  const long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (p >= P) return;
  const int e = idx[p];
  dest[p] = (e >= 0 && e < E) ? offsets[e] + atomicAdd(cursor + e, 1) : -1;   // -1: dropped by the row movers
}

// Expert-parallel plan.  allc [W][E] holds every rank's pick counts.  For expert e owned by rank
// e / El: start[e] = (first row of e inside its owner's receive buffer) + (rows that lower ranks
// send to e); offsets_local [El+1] are the padded segment boundaries of this rank's own experts;
// overflow is set when any owner would need more than `capacity` rows.  One CTA, E <= 1024.
__global__ void ep_plan_kernel(const int* __restrict__ allc, int* __restrict__ start, int* __restrict__ cursor,
                               int* __restrict__ offsets_local, int* __restrict__ overflow, int W, int E, int El,
                               int rank, int pad, int capacity) {
  __shared__ int sh[1024];
  const int t = threadIdx.x;
  int tot = 0, before = 0;
  if (t < E)
    for (int r = 0; r < W; ++r) {
      const int c = allc[r * E + t];
      if (r < rank) before += c;
      tot += c;
    }
  const int padded = (t < E) ? (tot + pad - 1) / pad * pad : 0;
  sh[t] = padded;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const int add = (t >= o) ? sh[t - o] : 0;
    __syncthreads();
    sh[t] += add;
    __syncthreads();
  }
  if (t < E) {
    const int owner_first = (t / El) * El;
    const int s0 = owner_first > 0 ? sh[owner_first - 1] : 0;
    start[t] = sh[t] - padded - s0 + before;
    cursor[t] = 0;
    if (t / El == rank) offsets_local[t - owner_first + 1] = sh[t] - s0;
    if (t % El == El - 1 && sh[t] - s0 > capacity) atomicExch(overflow, 1);
  }
  if (t == 0) offsets_local[0] = 0;
}

__global__ void ep_dest_kernel(const int* __restrict__ idx, const int* __restrict__ start, int* __restrict__ cursor,
                               int* __restrict__ dst_rank, int* __restrict__ dst_row, long long P, int El,
                               int capacity, int E) {
  const long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (p >= P) return;
  const int e = idx[p];
  if (e < 0 || e >= E) {  // never dereference an id that is out of range
    dst_rank[p] = 0;
    dst_row[p] = -1;
    return;
  }
  dst_rank[p] = e / El;
  const int row = start[e] + atomicAdd(cursor + e, 1);
  dst_row[p] = row < capacity ? row : -1;   // beyond the receive buffer: dropped (the overflow flag is set)
}

}  // namespace ob

using namespace ob;

extern "C" {

int ob_router_topk(const void* logits, float* probs, float* weights, int* idx, int* counts, long long M, int E, int k,
                   int renorm, cudaStream_t s) {
  if (E % 32 || E > 32 * kMaxEPL || E <= 0) return 6001;
  if (k <= 0 || k > kMaxTopK || k > E) return 6005;
  if (M <= 0) return 0;
  router_topk_kernel<<<(unsigned)((M * 32 + 255) / 256), 256, 0, s>>>((const bf16*)logits, probs, weights, idx, counts,
                                                                      M, E, k, renorm);
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_router_topk_bwd(const float* probs, const float* weights, const int* idx, const float* dweights,
                       const float* dprobs, void* dlogits, long long M, int E, int k, int renorm, cudaStream_t s) {
  if (E % 32 || E > 32 * kMaxEPL || E <= 0) return 6001;
  if (k <= 0 || k > kMaxTopK) return 6005;
  if (M <= 0) return 0;
  router_topk_bwd_kernel<<<(unsigned)((M * 32 + 255) / 256), 256, 0, s>>>(probs, weights, idx, dweights, dprobs,
                                                                          (bf16*)dlogits, M, E, k, renorm);
  OB_CHECK_LAUNCH();
  return 0;
}

// counts [E] -> offsets [E+1] and dest [P]; cursor is an E-int scratch.  With compute_counts the
// histogram of idx is taken here, otherwise counts must already hold it (e.g. from the router).
int ob_moe_plan(const int* idx, int* counts, int* offsets, int* cursor, int* dest, long long P, int E, int pad,
                int compute_counts, cudaStream_t s) {
  if (E > 1024 || E <= 0) return 6001;
  if (compute_counts) {
    cudaMemsetAsync(counts, 0, sizeof(int) * E, s);
    if (P > 0) moe_count_kernel<<<(unsigned)((P + 255) / 256), 256, 0, s>>>(idx, counts, P, E);
  }
  moe_offsets_kernel<<<1, 1024, 0, s>>>(counts, offsets, cursor, E, pad);
  OB_CHECK_LAUNCH();
  if (P > 0) {
    moe_dest_kernel<<<(unsigned)((P + 255) / 256), 256, 0, s>>>(idx, offsets, cursor, dest, P, E);
    OB_CHECK_LAUNCH();
  }
  return 0;
}

// counts[E] = histogram of idx (zeroed here first)
int ob_moe_count(const int* idx, int* counts, long long P, int E, cudaStream_t s) {
  cudaMemsetAsync(counts, 0, sizeof(int) * E, s);
  if (P > 0) {
    moe_count_kernel<<<(unsigned)((P + 255) / 256), 256, 0, s>>>(idx, counts, P, E);
    OB_CHECK_LAUNCH();
  }
  return 0;
}

// scratch: 2*E ints (start, cursor).  overflow is a sticky device flag.
int ob_ep_plan(const int* idx, const int* allc, int* scratch, int* offsets_local, int* dst_rank, int* dst_row,
               int* overflow, long long P, int W, int E, int rank, int pad, int capacity, cudaStream_t s) {
  if (E > 1024 || E <= 0 || W <= 0 || E % W) return 6001;
  const int El = E / W;
  ep_plan_kernel<<<1, 1024, 0, s>>>(allc, scratch, scratch + E, offsets_local, overflow, W, E, El, rank, pad, capacity);
  OB_CHECK_LAUNCH();
  if (P > 0) {
    ep_dest_kernel<<<(unsigned)((P + 255) / 256), 256, 0, s>>>(idx, scratch, scratch + E, dst_rank, dst_row, P, El, capacity, E);
    OB_CHECK_LAUNCH();
  }
  return 0;
}

}  // extern "C"
