// K7b: causal depthwise conv1d (kernel width <= 4) + SiLU over [B, T, C] bf16, forward and
// backward, for the GatedDeltaNet input mixing.  y[b,t,c] = silu(sum_j w[c,j] * x[b,t-KW+1+j,c])
// with zeros left of t = 0.  One thread handles 8 channels over a run of 32 time steps and keeps
// the sliding window in registers; weight gradients are reduced per thread and added with
// fp32 atomics.
#include "host_utils.h"
#include "sm100_common.cuh"

namespace ob {

constexpr int kRun = 32;

__device__ __forceinline__ void load8(const bf16* p, float* f) {
  uint4 q = *reinterpret_cast<const uint4*>(p);
  uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 t = unpack_bf16(u[j]);
    f[2 * j] = t.x; f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(bf16* p, const float* f) {
  uint4 q;
  q.x = pack_bf16(f[0], f[1]); q.y = pack_bf16(f[2], f[3]);
  q.z = pack_bf16(f[4], f[5]); q.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = q;
}

template <int KW>
__global__ void conv1d_silu_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                       bf16* __restrict__ y, int B, int T, int C) {
  const int cv = C >> 3;
  const int runs = (T + kRun - 1) / kRun;
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)B * runs * cv) return;
  const int c8 = (int)(idx % cv);
  const int run = (int)((idx / cv) % runs);
  const int b = (int)(idx / ((long long)cv * runs));
  const int c0 = c8 * 8;
  float wv[8][KW];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < KW; ++j) wv[i][j] = __bfloat162float(w[(c0 + i) * KW + j]);
  const int t0 = run * kRun, t1 = min(T, t0 + kRun);
  float win[KW][8];  // win[j] = x at time t-KW+1+j
#pragma unroll
  for (int j = 0; j < KW - 1; ++j) {
    const int t = t0 - (KW - 1) + j;
    if (t >= 0) load8(x + ((long long)b * T + t) * C + c0, win[j + 1]);
    else
#pragma unroll
      for (int i = 0; i < 8; ++i) win[j + 1][i] = 0.f;
  }
  for (int t = t0; t < t1; ++t) {
#pragma unroll
    for (int j = 0; j < KW - 1; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) win[j][i] = win[j + 1][i];
    load8(x + ((long long)b * T + t) * C + c0, win[KW - 1]);
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float a = 0.f;
#pragma unroll
      for (int j = 0; j < KW; ++j) a += wv[i][j] * win[j][i];
      o[i] = a / (1.f + __expf(-a));
    }
    store8(y + ((long long)b * T + t) * C + c0, o);
  }
}

// dpre[t] = dy[t] * silu'(pre[t]);  dx[t] = sum_j w[j] * dpre[t + KW-1-j];  dw[j] += dpre[t] * x[t-KW+1+j]
// One thread walks a run of kRun time steps of two channels with sliding windows: x[t-3 .. t+3] and
// dpre[t .. t+3] live in registers, so a step costs one x load, one dy load, one sigmoid and one
// store (the first version re-derived every dpre four times: 24 loads and 4 sigmoids per step).
// A warp covers 64 consecutive channels (128 bytes) per access.
template <int KW>
__global__ void conv1d_silu_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                       const bf16* __restrict__ dy, bf16* __restrict__ dx,
                                       float* __restrict__ dw, int B, int T, int C) {
  static_assert(KW == 4, "window arithmetic below is written for four taps");
  constexpr int CPT = 2;
  const int cv = C / CPT;
  const int runs = (T + kRun - 1) / kRun;
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)B * runs * cv) return;
  const int cg = (int)(idx % cv);
  const int run = (int)((idx / cv) % runs);
  const int b = (int)(idx / ((long long)cv * runs));
  const int c0 = cg * CPT;
  float wv[CPT][KW], dwv[CPT][KW];
#pragma unroll
  for (int i = 0; i < CPT; ++i)
#pragma unroll
    for (int j = 0; j < KW; ++j) { wv[i][j] = __bfloat162float(w[(c0 + i) * KW + j]); dwv[i][j] = 0.f; }
  const int t0 = run * kRun, t1 = min(T, t0 + kRun);
  const bf16* xb = x + (long long)b * T * C + c0;
  const bf16* gb = dy + (long long)b * T * C + c0;
  auto ld2 = [&](const bf16* base, int t, float* f) {   // two channels of time step t, zero outside [0, T)
    if (t >= 0 && t < T) {
      const float2 v = unpack_bf16(*reinterpret_cast<const uint32_t*>(base + (long long)t * C));
      f[0] = v.x; f[1] = v.y;
    } else {
      f[0] = f[1] = 0.f;
    }
  };
  float xw[7][CPT];   // x[t-3 .. t+3]
  float dp[4][CPT];   // dpre[t .. t+3]
#pragma unroll
  for (int o = 0; o < 6; ++o) ld2(xb, t0 - 3 + o, xw[o]);
  auto dpre_from = [&](const float (*xs)[CPT], int t, float* out) {   // xs[0..3] = x[t-3 .. t]
    float g[CPT];
    ld2(gb, t, g);
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      float pre = 0.f;
#pragma unroll
      for (int j = 0; j < KW; ++j) pre += wv[i][j] * xs[j][i];
      const float sg = 1.f / (1.f + __expf(-pre));
      out[i] = (t < T) ? g[i] * sg * (1.f + pre * (1.f - sg)) : 0.f;
    }
  };
#pragma unroll
  for (int o = 0; o < 3; ++o) dpre_from(&xw[o], t0 + o, dp[o]);
  for (int t = t0; t < t1; ++t) {
    ld2(xb, t + 3, xw[6]);
    dpre_from(&xw[3], t + 3, dp[3]);
    float acc[CPT];
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      acc[i] = 0.f;
#pragma unroll
      for (int j = 0; j < KW; ++j) acc[i] += wv[i][j] * dp[KW - 1 - j][i];
#pragma unroll
      for (int jj = 0; jj < KW; ++jj) dwv[i][jj] += dp[0][i] * xw[jj][i];   // x[t-3+jj]
    }
    *reinterpret_cast<uint32_t*>(dx + ((long long)b * T + t) * C + c0) = pack_bf16(acc[0], acc[1]);
#pragma unroll
    for (int o = 0; o < 6; ++o)
#pragma unroll
      for (int i = 0; i < CPT; ++i) xw[o][i] = xw[o + 1][i];
#pragma unroll
    for (int o = 0; o < 3; ++o)
#pragma unroll
      for (int i = 0; i < CPT; ++i) dp[o][i] = dp[o + 1][i];
  }
  if (dw) {
#pragma unroll
    for (int i = 0; i < CPT; ++i)
#pragma unroll
      for (int j = 0; j < KW; ++j) atomicAdd(dw + (c0 + i) * KW + j, dwv[i][j]);
  }
}

}  // namespace ob

using namespace ob;

extern "C" {

int ob_conv1d_silu_fwd(const void* x, const void* w, void* y, int B, int T, int C, int KW, cudaStream_t s) {
  if (C % 8) return 6001;
  if (KW != 4) return 6005;
  long long n = (long long)B * ((T + kRun - 1) / kRun) * (C / 8);
  if (n <= 0) return 0;
  conv1d_silu_fwd_kernel<4><<<(unsigned)((n + 127) / 128), 128, 0, s>>>((const bf16*)x, (const bf16*)w, (bf16*)y, B, T, C);
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_conv1d_silu_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw, int B, int T, int C,
                       int KW, cudaStream_t s) {
  if (C % 8) return 6001;
  if (KW != 4) return 6005;
  long long n = (long long)B * ((T + kRun - 1) / kRun) * (C / 2);
  if (n <= 0) return 0;
  conv1d_silu_bwd_kernel<4><<<(unsigned)((n + 127) / 128), 128, 0, s>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy,
                                                                        (bf16*)dx, dw, B, T, C);
  OB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
