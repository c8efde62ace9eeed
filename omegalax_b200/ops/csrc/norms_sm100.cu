// Gated RMSNorm (GatedDeltaNet output norm) and LayerNorm with bias (vision tower), forward and
// backward.  One warp per row, fp32 statistics, 128-bit accesses; the parameter gradients are
// reduced per warp over a strided set of rows, then across the CTA in shared memory, then added
// to an fp32 buffer with atomics.
//
// Gated RMSNorm numerics follow omegalax/models/qwen3_5/norms.py:52-60: normalise in fp32, cast,
// multiply by the weight in the model dtype, multiply by silu(z) evaluated in fp32, cast.
#include "host_utils.h"
#include "sm100_common.cuh"

namespace ob {

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

__device__ __forceinline__ void ld4(const bf16* p, float* f) {
  const uint2 q = *reinterpret_cast<const uint2*>(p);
  const float2 a = unpack_bf16(q.x), b = unpack_bf16(q.y);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void st4(bf16* p, const float* f) {
  uint2 q;
  q.x = pack_bf16(f[0], f[1]);
  q.y = pack_bf16(f[2], f[3]);
  *reinterpret_cast<uint2*>(p) = q;
}

// ----------------------------------------------------------------------------- gated RMSNorm
// D = 128 * NV; lane handles elements 4*lane + 128*i.
template <int NV>
__global__ void gated_rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ z,
                                         const bf16* __restrict__ w, bf16* __restrict__ y,
                                         float* __restrict__ rstd_out, long long M, float eps) {
  constexpr int D = 128 * NV;
  const int lane = threadIdx.x & 31;
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (row >= M) return;
  float xv[NV][4], wv[NV][4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    ld4(x + row * D + 128 * i + 4 * lane, xv[i]);
    ld4(w + 128 * i + 4 * lane, wv[i]);
#pragma unroll
    for (int e = 0; e < 4; ++e) ss = fmaf(xv[i][e], xv[i][e], ss);
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / D + eps);
  if (lane == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float zv[4], o[4];
    ld4(z + row * D + 128 * i + 4 * lane, zv);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float n = bf16_round(xv[i][e] * rstd);
      const float n2 = bf16_round(wv[i][e] * n);
      o[e] = n2 * (zv[e] / (1.f + __expf(-zv[e])));
    }
    st4(y + row * D + 128 * i + 4 * lane, o);
  }
}

template <int NV>
__global__ void gated_rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                         const bf16* __restrict__ z, const bf16* __restrict__ w,
                                         const float* __restrict__ rstd_in, bf16* __restrict__ dx,
                                         bf16* __restrict__ dz, float* __restrict__ dw, long long M, float eps) {
  constexpr int D = 128 * NV;
  __shared__ float red[8][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  float wv[NV][4], dwv[NV][4];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    ld4(w + 128 * i + 4 * lane, wv[i]);
#pragma unroll
    for (int e = 0; e < 4; ++e) dwv[i][e] = 0.f;
  }
  for (long long row = blockIdx.x * (long long)(blockDim.x >> 5) + warp; row < M; row += nwarps) {
    float xv[NV][4], dn[NV][4];
    float rstd;
    if (rstd_in) {
      rstd = rstd_in[row];
#pragma unroll
      for (int i = 0; i < NV; ++i) ld4(x + row * D + 128 * i + 4 * lane, xv[i]);
    } else {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        ld4(x + row * D + 128 * i + 4 * lane, xv[i]);
#pragma unroll
        for (int e = 0; e < 4; ++e) ss = fmaf(xv[i][e], xv[i][e], ss);
      }
      rstd = rsqrtf(warp_sum(ss) / D + eps);
    }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float zv[4], g[4], dzv[4];
      ld4(z + row * D + 128 * i + 4 * lane, zv);
      ld4(dy + row * D + 128 * i + 4 * lane, g);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float xh = xv[i][e] * rstd;
        const float n = bf16_round(xh);
        const float n2 = bf16_round(wv[i][e] * n);
        const float sg = 1.f / (1.f + __expf(-zv[e]));
        const float dt = g[e] * zv[e] * sg;                       // d(w * n)
        dzv[e] = g[e] * n2 * sg * (1.f + zv[e] * (1.f - sg));
        dwv[i][e] = fmaf(dt, n, dwv[i][e]);
        dn[i][e] = dt * wv[i][e];
        dot = fmaf(dn[i][e], xh, dot);
        xv[i][e] = xh;
      }
      st4(dz + row * D + 128 * i + 4 * lane, dzv);
    }
    dot = warp_sum(dot) / D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = rstd * (dn[i][e] - xv[i][e] * dot);
      st4(dx + row * D + 128 * i + 4 * lane, o);
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) red[warp][128 * i + 4 * lane + e] = dwv[i][e];
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float s = 0.f;
    for (int wi = 0; wi < (int)(blockDim.x >> 5); ++wi) s += red[wi][d];
    atomicAdd(dw + d, s);
  }
}

// ----------------------------------------------------------------------------- LayerNorm
// lane handles elements 8*lane + 256*i, i < NV; D <= 256 * NV, D % 8 == 0.
__device__ __forceinline__ void ld8(const bf16* p, float* f) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = unpack_bf16(u[j]);
    f[2 * j] = t.x; f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ void st8(bf16* p, const float* f) {
  uint4 q;
  q.x = pack_bf16(f[0], f[1]); q.y = pack_bf16(f[2], f[3]);
  q.z = pack_bf16(f[4], f[5]); q.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = q;
}

template <int NV>
__global__ void layernorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                     const bf16* __restrict__ b, bf16* __restrict__ y,
                                     float* __restrict__ mean_out, float* __restrict__ rstd_out, long long M, int D,
                                     float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (row >= M) return;
  float xv[NV][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 8 * lane + 256 * i;
    if (c < D) {
      ld8(x + row * D + c, xv[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) s += xv[i][e];
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) xv[i][e] = 0.f;
    }
  }
  const float mean = warp_sum(s) / D;
  float var = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i)
    if (8 * lane + 256 * i < D)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float c = xv[i][e] - mean;
        var = fmaf(c, c, var);
      }
  const float rstd = rsqrtf(warp_sum(var) / D + eps);
  if (lane == 0 && mean_out) { mean_out[row] = mean; rstd_out[row] = rstd; }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 8 * lane + 256 * i;
    if (c < D) {
      float wv[8], bv[8], o[8];
      ld8(w + c, wv);
      ld8(b + c, bv);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = fmaf((xv[i][e] - mean) * rstd, wv[e], bv[e]);
      st8(y + row * D + c, o);
    }
  }
}

template <int NV>
__global__ void layernorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                     const bf16* __restrict__ w, const float* __restrict__ mean_in,
                                     const float* __restrict__ rstd_in, bf16* __restrict__ dx,
                                     float* __restrict__ dw, float* __restrict__ db, long long M, int D) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  float wv[NV][8], dwv[NV][8], dbv[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 8 * lane + 256 * i;
    if (c < D) ld8(w + c, wv[i]);
#pragma unroll
    for (int e = 0; e < 8; ++e) { dwv[i][e] = 0.f; dbv[i][e] = 0.f; if (c >= D) wv[i][e] = 0.f; }
  }
  for (long long row = blockIdx.x * (long long)(blockDim.x >> 5) + warp; row < M; row += nwarps) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[NV][8], g[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = 8 * lane + 256 * i;
      if (c < D) {
        float gy[8];
        ld8(x + row * D + c, xh[i]);
        ld8(dy + row * D + c, gy);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[i][e] = (xh[i][e] - mean) * rstd;
          dwv[i][e] = fmaf(gy[e], xh[i][e], dwv[i][e]);
          dbv[i][e] += gy[e];
          g[i][e] = gy[e] * wv[i][e];
          s1 += g[i][e];
          s2 = fmaf(g[i][e], xh[i][e], s2);
        }
      }
    }
    s1 = warp_sum(s1) / D;
    s2 = warp_sum(s2) / D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = 8 * lane + 256 * i;
      if (c < D) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rstd * (g[i][e] - s1 - xh[i][e] * s2);
        st8(dx + row * D + c, o);
      }
    }
  }
  // per-column sums: first over the 8 warps of the CTA in shared memory (one 256-column slice at a
  // time), then one atomic per column and CTA (the earlier version issued one per column and warp:
  // 2 x D x 8 x CTAs atomics on 2 x D addresses, which dominated the kernel on short inputs)
  __shared__ float red_w[8][256], red_b[8][256];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      red_w[warp][8 * lane + e] = dwv[i][e];
      red_b[warp][8 * lane + e] = dbv[i][e];
    }
    __syncthreads();
    const int c = 256 * i + threadIdx.x;      // blockDim.x == 256
    if (c < D) {
      float sw = 0.f, sb = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) { sw += red_w[q][threadIdx.x]; sb += red_b[q][threadIdx.x]; }
      atomicAdd(dw + c, sw);
      atomicAdd(db + c, sb);
    }
    __syncthreads();
  }
}

}  // namespace ob

using namespace ob;

extern "C" {

int ob_gated_rmsnorm_fwd(const void* x, const void* z, const void* w, void* y, float* rstd, long long M, int D,
                         float eps, cudaStream_t s) {
  if (M <= 0) return 0;
  const unsigned blocks = (unsigned)((M * 32 + 255) / 256);
  if (D == 128) gated_rmsnorm_fwd_kernel<1><<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)z, (const bf16*)w, (bf16*)y, rstd, M, eps);
  else if (D == 256) gated_rmsnorm_fwd_kernel<2><<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)z, (const bf16*)w, (bf16*)y, rstd, M, eps);
  else return 6001;
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_gated_rmsnorm_bwd(const void* dy, const void* x, const void* z, const void* w, const float* rstd, void* dx,
                         void* dz, float* dw, long long M, int D, float eps, cudaStream_t s) {
  if (M <= 0) return 0;
  long long want = (M + 7) / 8;
  const unsigned blocks = (unsigned)(want < (long long)num_sms() * 8 ? want : (long long)num_sms() * 8);
  if (D == 128) gated_rmsnorm_bwd_kernel<1><<<blocks, 256, 0, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)z, (const bf16*)w, rstd, (bf16*)dx, (bf16*)dz, dw, M, eps);
  else if (D == 256) gated_rmsnorm_bwd_kernel<2><<<blocks, 256, 0, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)z, (const bf16*)w, rstd, (bf16*)dx, (bf16*)dz, dw, M, eps);
  else return 6001;
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, long long M,
                     int D, float eps, cudaStream_t s) {
  if (M <= 0) return 0;
  if (D % 8 || D > 2048) return 6001;
  const unsigned blocks = (unsigned)((M * 32 + 255) / 256);
#define OB_LN_FWD(NV) layernorm_fwd_kernel<NV><<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)w, (const bf16*)b, (bf16*)y, mean, rstd, M, D, eps)
  if (D <= 1024) OB_LN_FWD(4);
  else if (D <= 1536) OB_LN_FWD(6);
  else OB_LN_FWD(8);
#undef OB_LN_FWD
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                     float* dw, float* db, long long M, int D, cudaStream_t s) {
  if (M <= 0) return 0;
  if (D % 8 || D > 2048) return 6001;
  long long want = (M + 7) / 8;
  const unsigned blocks = (unsigned)(want < (long long)num_sms() ? want : (long long)num_sms());
#define OB_LN_BWD(NV) layernorm_bwd_kernel<NV><<<blocks, 256, 0, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, mean, rstd, (bf16*)dx, dw, db, M, D)
  if (D <= 1024) OB_LN_BWD(4);
  else if (D <= 1536) OB_LN_BWD(6);
  else OB_LN_BWD(8);
#undef OB_LN_BWD
  OB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
