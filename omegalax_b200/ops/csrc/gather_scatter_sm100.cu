// K13: small row gather / scatter kernels and the tanh-GELU of the vision MLP.
//   gather_rows        out[i, :] = src[idx[i], :]
//   scatter_rows       dst[idx[i], :] (+)= src[i, :]          (idx unique: image-token positions)
//   gather4 fwd / bwd  out[i, :] = sum_k w[i,k] * table[idx[i,k], :]   (bilinear position-embedding
//                      lookup: four neighbours per output row); backward adds into an fp32 table
//   gelu_tanh fwd/bwd  0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
// All rows are bf16 with D a multiple of 8 (16-byte accesses).
#include "host_utils.h"
#include "sm100_common.cuh"

namespace ob {

__device__ __forceinline__ void u4_to_f8(const uint4& q, float* f) {
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = unpack_bf16(u[j]);
    f[2 * j] = t.x; f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 f8_to_u4(const float* f) {
  uint4 q;
  q.x = pack_bf16(f[0], f[1]); q.y = pack_bf16(f[2], f[3]);
  q.z = pack_bf16(f[4], f[5]); q.w = pack_bf16(f[6], f[7]);
  return q;
}

__global__ void gather_rows_kernel(const bf16* __restrict__ src, const int* __restrict__ idx, bf16* __restrict__ out,
                                   long long n, int D) {
  const int dv = D >> 3;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < n * dv; t += (long long)gridDim.x * blockDim.x) {
    const long long i = t / dv;
    const int c = (int)(t - i * dv);
    reinterpret_cast<uint4*>(out + i * D)[c] = reinterpret_cast<const uint4*>(src + (long long)idx[i] * D)[c];
  }
}

__global__ void scatter_rows_kernel(bf16* __restrict__ dst, const int* __restrict__ idx, const bf16* __restrict__ src,
                                    long long n, int D, int replace) {
  const int dv = D >> 3;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < n * dv; t += (long long)gridDim.x * blockDim.x) {
    const long long i = t / dv;
    const int c = (int)(t - i * dv);
    uint4* d = reinterpret_cast<uint4*>(dst + (long long)idx[i] * D) + c;
    const uint4 s = reinterpret_cast<const uint4*>(src + i * D)[c];
    if (replace) {
      *d = s;
    } else {
      float a[8], b[8];
      u4_to_f8(*d, a);
      u4_to_f8(s, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
      *d = f8_to_u4(a);
    }
  }
}

__global__ void gather4_fwd_kernel(const bf16* __restrict__ table, const int* __restrict__ idx,
                                   const float* __restrict__ w, bf16* __restrict__ out, long long n, int D) {
  const int dv = D >> 3;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < n * dv; t += (long long)gridDim.x * blockDim.x) {
    const long long i = t / dv;
    const int c = (int)(t - i * dv);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float f[8];
      u4_to_f8(reinterpret_cast<const uint4*>(table + (long long)idx[i * 4 + k] * D)[c], f);
      const float wk = w[i * 4 + k];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(wk, f[j], acc[j]);
    }
    reinterpret_cast<uint4*>(out + i * D)[c] = f8_to_u4(acc);
  }
}

__global__ void gather4_bwd_kernel(const bf16* __restrict__ dout, const int* __restrict__ idx,
                                   const float* __restrict__ w, float* __restrict__ dtable, long long n, int D) {
  const int dv = D >> 3;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < n * dv; t += (long long)gridDim.x * blockDim.x) {
    const long long i = t / dv;
    const int c = (int)(t - i * dv);
    float g[8];
    u4_to_f8(reinterpret_cast<const uint4*>(dout + i * D)[c], g);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float* dst = dtable + (long long)idx[i * 4 + k] * D + c * 8;
      const float wk = w[i * 4 + k];
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(dst + j, wk * g[j]);
    }
  }
}

__device__ __forceinline__ float gelu_t(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}
__device__ __forceinline__ float gelu_t_grad(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  const float th = tanhf(u);
  const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
  return 0.5f * (1.f + th) + 0.5f * x * (1.f - th * th) * du;
}

__global__ void gelu_tanh_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long nv) {
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nv; t += (long long)gridDim.x * blockDim.x) {
    float f[8];
    u4_to_f8(reinterpret_cast<const uint4*>(x)[t], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = gelu_t(f[j]);
    reinterpret_cast<uint4*>(y)[t] = f8_to_u4(f);
  }
}
__global__ void gelu_tanh_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, bf16* __restrict__ dx,
                                     long long nv) {
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nv; t += (long long)gridDim.x * blockDim.x) {
    float f[8], g[8];
    u4_to_f8(reinterpret_cast<const uint4*>(x)[t], f);
    u4_to_f8(reinterpret_cast<const uint4*>(dy)[t], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= gelu_t_grad(f[j]);
    reinterpret_cast<uint4*>(dx)[t] = f8_to_u4(g);
  }
}

static unsigned blocks_for(long long work) {
  long long b = (work + 255) / 256;
  const long long cap = (long long)num_sms() * 16;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace ob

using namespace ob;

extern "C" {

int ob_gather_rows(const void* src, const int* idx, void* out, long long n, int D, cudaStream_t s) {
  if (D % 8) return 6001;
  if (n <= 0) return 0;
  gather_rows_kernel<<<blocks_for(n * (D / 8)), 256, 0, s>>>((const bf16*)src, idx, (bf16*)out, n, D);
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_scatter_rows(void* dst, const int* idx, const void* src, long long n, int D, int replace, cudaStream_t s) {
  if (D % 8) return 6001;
  if (n <= 0) return 0;
  scatter_rows_kernel<<<blocks_for(n * (D / 8)), 256, 0, s>>>((bf16*)dst, idx, (const bf16*)src, n, D, replace);
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_gather4_fwd(const void* table, const int* idx, const float* w, void* out, long long n, int D, cudaStream_t s) {
  if (D % 8) return 6001;
  if (n <= 0) return 0;
  gather4_fwd_kernel<<<blocks_for(n * (D / 8)), 256, 0, s>>>((const bf16*)table, idx, w, (bf16*)out, n, D);
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_gather4_bwd(const void* dout, const int* idx, const float* w, float* dtable, long long n, int D, cudaStream_t s) {
  if (D % 8) return 6001;
  if (n <= 0) return 0;
  gather4_bwd_kernel<<<blocks_for(n * (D / 8)), 256, 0, s>>>((const bf16*)dout, idx, w, dtable, n, D);
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_gelu_tanh_fwd(const void* x, void* y, long long n, cudaStream_t s) {
  if (n % 8) return 6001;
  if (n <= 0) return 0;
  gelu_tanh_fwd_kernel<<<blocks_for(n / 8), 256, 0, s>>>((const bf16*)x, (bf16*)y, n / 8);
  OB_CHECK_LAUNCH();
  return 0;
}

int ob_gelu_tanh_bwd(const void* x, const void* dy, void* dx, long long n, cudaStream_t s) {
  if (n % 8) return 6001;
  if (n <= 0) return 0;
  gelu_tanh_bwd_kernel<<<blocks_for(n / 8), 256, 0, s>>>((const bf16*)x, (const bf16*)dy, (bf16*)dx, n / 8);
  OB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
