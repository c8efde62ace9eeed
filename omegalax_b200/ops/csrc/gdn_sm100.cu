// K7a: chunked gated delta rule (GatedDeltaNet core), forward and backward, fp32 throughout
// (the reference keeps this recurrence in fp32: omegalax/models/qwen3_5/deltanet.py:68-70).
//
// Per (batch, value head) the state S [A=128, U] is carried through the sequence in chunks of
// 64 tokens.  With gamma = cumsum(g) inside the chunk, a_i = exp(gamma_i), b_j = exp(gamma_C - gamma_j),
// D_ij = exp(gamma_i - gamma_j):
//     L_ij = beta_i (k_i . k_j) D_ij  (i > j)        P_ij = (q_i . k_j) D_ij  (i >= j)
//     r_i  = beta_i (v_i - a_i (k S)_i)              (I + L) n = r            (forward substitution)
//     o_i  = a_i (q S)_i + sum_j P_ij n_j            S'  = a_C S + sum_j b_j k_j n_j^T
// The backward walks the chunks in reverse with dS in shared memory, re-using the chunk-start
// states and the solved rows n that the forward saved:
//     dn = P^T do + b (k dS')        (I + L)^T dr = dn        dL = -dr n^T     dP = do n^T
// and everything else follows by the product rule (see the phase comments in the kernel).
//
// One CTA of 256 threads owns one (batch, head, slice of U).  All matrix products run through
// one register-tiled routine over padded shared-memory tiles (row strides = 4 mod 32 words, so
// both row-wise and column-wise 128-bit reads are conflict free).  U slices are independent in
// the forward; in the backward the quantities that sum over U (dq, dk, dg, dbeta) are linear in
// the per-slice partial sums and are accumulated with vector fp32 reductions in global memory.
#include "host_utils.h"
#include "sm100_common.cuh"

namespace ob {

constexpr int GC = 64;     // chunk length
constexpr int GA = 128;    // key head dim
constexpr int LDA_ = GA + 4;
constexpr int LDC_ = GC + 4;

struct GdnArgs {
  const float* q;       // [B,T,Hk,A]  (L2-normalised, q pre-scaled)
  const float* k;       // [B,T,Hk,A]
  const float* v;       // [B,T,H,U]
  const float* g;       // [B,T,H]   log decay (<= 0)
  const float* beta;    // [B,T,H]
  const float* s0;      // [B,H,A,U] or null
  float* o;             // [B,T,H,U]
  float* n_out;         // [B,T,H,U] solved rows (saved for the backward) or null
  float* states;        // [B,H,J,A,U] chunk-start states or null
  float* s_final;       // [B,H,A,U] or null
  // backward only
  const float* d_o;     // [B,T,H,U]
  const float* d_sfinal;// [B,H,A,U] or null
  float* dq;            // [B,T,Hk,A]  accumulated (zero-initialised by the caller)
  float* dk;            // [B,T,Hk,A]  accumulated
  float* dv;            // [B,T,H,U]
  float* dg;            // [B,T,H]     accumulated
  float* dbeta;         // [B,T,H]     accumulated
  float* ds0;           // [B,H,A,U] or null
  int B, T, H, Hk, U;   // T is a multiple of 64
};

// Index of accumulator row c for the operand that is addressed by ty (always groups of four
// consecutive indices), and of column d for the operand addressed by tx.
__device__ __forceinline__ int mi(int c, int ty) { return 64 * (c >> 2) + 4 * ty + (c & 3); }
template <bool KMAJ>
__device__ __forceinline__ int ni(int d, int tx) {
  return KMAJ ? 64 * (d >> 2) + 4 * tx + (d & 3) : tx + 16 * d;
}

// acc[c][d] += sum_k A(mi(c), k) * B(k, ni(d)) * kscale[k].
//   A_KMAJ: A is stored [k][m] (row stride lda), else [m][k].   B likewise with n.
// K is a multiple of 4; all tiles are 16-byte aligned with strides that are multiples of 4.
template <int TM, int TN, bool A_KMAJ, bool B_KMAJ>
__device__ __forceinline__ void mm(float (&acc)[TM][TN], const float* __restrict__ A, int lda,
                                   const float* __restrict__ Bm, int ldb, int K, int ty, int tx,
                                   const float* __restrict__ kscale = nullptr) {
#pragma unroll 1
  for (int k = 0; k < K; k += 4) {
    float a[4][TM], b[4][TN];
    if (A_KMAJ) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
#pragma unroll
        for (int gq = 0; gq < TM / 4; ++gq) {
          const float4 t = *reinterpret_cast<const float4*>(A + (k + kk) * lda + 64 * gq + 4 * ty);
          a[kk][4 * gq + 0] = t.x; a[kk][4 * gq + 1] = t.y; a[kk][4 * gq + 2] = t.z; a[kk][4 * gq + 3] = t.w;
        }
    } else {
#pragma unroll
      for (int c = 0; c < TM; ++c) {
        const float4 t = *reinterpret_cast<const float4*>(A + mi(c, ty) * lda + k);
        a[0][c] = t.x; a[1][c] = t.y; a[2][c] = t.z; a[3][c] = t.w;
      }
    }
    if (B_KMAJ) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
#pragma unroll
        for (int gq = 0; gq < TN / 4; ++gq) {
          const float4 t = *reinterpret_cast<const float4*>(Bm + (k + kk) * ldb + 64 * gq + 4 * tx);
          b[kk][4 * gq + 0] = t.x; b[kk][4 * gq + 1] = t.y; b[kk][4 * gq + 2] = t.z; b[kk][4 * gq + 3] = t.w;
        }
    } else {
#pragma unroll
      for (int d = 0; d < TN; ++d) {
        const float4 t = *reinterpret_cast<const float4*>(Bm + (tx + 16 * d) * ldb + k);
        b[0][d] = t.x; b[1][d] = t.y; b[2][d] = t.z; b[3][d] = t.w;
      }
    }
    if (kscale) {
      const float4 s = *reinterpret_cast<const float4*>(kscale + k);
#pragma unroll
      for (int c = 0; c < TM; ++c) { a[0][c] *= s.x; a[1][c] *= s.y; a[2][c] *= s.z; a[3][c] *= s.w; }
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
#pragma unroll
      for (int c = 0; c < TM; ++c)
#pragma unroll
        for (int d = 0; d < TN; ++d) acc[c][d] = fmaf(a[kk][c], b[kk][d], acc[c][d]);
  }
}

template <int TM, int TN>
__device__ __forceinline__ void zero(float (&acc)[TM][TN]) {
#pragma unroll
  for (int c = 0; c < TM; ++c)
#pragma unroll
    for (int d = 0; d < TN; ++d) acc[c][d] = 0.f;
}

// sum over the 16 lanes that share ty (a half warp)
__device__ __forceinline__ float half_warp_sum(float x) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Loads the 64 x 128 rows of one chunk of q or k (row stride Hk*A floats in global memory).
__device__ __forceinline__ void load_rows128(float* dst, const float* src, long long row_stride, int tid) {
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int idx = tid + 256 * it;
    const int r = idx >> 5, c4 = idx & 31;
    *reinterpret_cast<float4*>(dst + r * LDA_ + 4 * c4) = *reinterpret_cast<const float4*>(src + r * row_stride + 4 * c4);
  }
}
// Loads a 64 x UB slice (row stride H*U floats).
template <int UB>
__device__ __forceinline__ void load_rowsU(float* dst, const float* src, long long row_stride, int tid) {
  constexpr int V = UB / 4;
  for (int idx = tid; idx < GC * V; idx += 256) {
    const int r = idx / V, c4 = idx % V;
    *reinterpret_cast<float4*>(dst + r * (UB + 4) + 4 * c4) = *reinterpret_cast<const float4*>(src + r * row_stride + 4 * c4);
  }
}
// State tile [128][UB] <-> global [128][U] slice.
template <int UB>
__device__ __forceinline__ void load_state(float* dst, const float* src, int U, int tid) {
  constexpr int V = UB / 4;
  for (int idx = tid; idx < GA * V; idx += 256) {
    const int r = idx / V, c4 = idx % V;
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
    if (src) t = *reinterpret_cast<const float4*>(src + (long long)r * U + 4 * c4);
    *reinterpret_cast<float4*>(dst + r * (UB + 4) + 4 * c4) = t;
  }
}
template <int UB>
__device__ __forceinline__ void store_state(float* dst, const float* src, int U, int tid) {
  constexpr int V = UB / 4;
  for (int idx = tid; idx < GA * V; idx += 256) {
    const int r = idx / V, c4 = idx % V;
    *reinterpret_cast<float4*>(dst + (long long)r * U + 4 * c4) = *reinterpret_cast<const float4*>(src + r * (UB + 4) + 4 * c4);
  }
}

// gamma (inclusive cumsum of g), a = exp(gamma), b = exp(gamma_last - gamma); one warp.
__device__ __forceinline__ void chunk_scalars(const float* g_s, float* gam_s, float* a_s, float* b_s, int tid) {
  if (tid < 32) {
    float x0 = g_s[2 * tid], x1 = g_s[2 * tid + 1];
    float s = x0 + x1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, s, o);
      if (tid >= o) s += t;
    }
    const float g1 = s, g0 = s - x1;
    const float last = __shfl_sync(0xffffffffu, s, 31);
    gam_s[2 * tid] = g0; gam_s[2 * tid + 1] = g1;
    a_s[2 * tid] = expf(g0); a_s[2 * tid + 1] = expf(g1);
    b_s[2 * tid] = expf(last - g0); b_s[2 * tid + 1] = expf(last - g1);
  }
}

// ----------------------------------------------------------------------------- forward
template <int UB>
__global__ void __launch_bounds__(256, 1) gdn_fwd_kernel(GdnArgs p) {
  constexpr int LDU = UB + 4;
  constexpr int TNU = UB / 16;
  constexpr int NS = GA / UB;
  extern __shared__ __align__(16) float gsm[];
  float* S_s = gsm;                   // [128][LDU]
  float* k_s = S_s + GA * LDU;        // [64][132]
  float* q_s = k_s + GC * LDA_;       // [64][132]
  float* n_s = q_s + GC * LDA_;       // [64][LDU]   v -> r -> n
  float* L_s = n_s + GC * LDU;        // [64][68]
  float* P_s = L_s + GC * LDC_;       // [64][68]
  float* g_s = P_s + GC * LDC_;       // 64 each below
  float* beta_s = g_s + GC;
  float* gam_s = beta_s + GC;
  float* a_s = gam_s + GC;
  float* b_s = a_s + GC;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int bh = blockIdx.x / NS, us = blockIdx.x % NS;
  const int b = bh / p.H, h = bh % p.H, hk = h / (p.H / p.Hk);
  const int u0 = us * UB, U = p.U, T = p.T, J = T / GC;
  const long long qk_stride = (long long)p.Hk * GA, v_stride = (long long)p.H * U;

  load_state<UB>(S_s, p.s0 ? p.s0 + (long long)bh * GA * U + u0 : nullptr, U, tid);
  __syncthreads();

  for (int j = 0; j < J; ++j) {
    const long long row0 = (long long)b * T + (long long)j * GC;
    load_rows128(k_s, p.k + (row0 * p.Hk + hk) * GA, qk_stride, tid);
    load_rows128(q_s, p.q + (row0 * p.Hk + hk) * GA, qk_stride, tid);
    load_rowsU<UB>(n_s, p.v + (row0 * p.H + h) * U + u0, v_stride, tid);
    if (tid < GC) {
      g_s[tid] = p.g[(row0 + tid) * p.H + h];
      beta_s[tid] = p.beta[(row0 + tid) * p.H + h];
    }
    if (p.states) store_state<UB>(p.states + ((long long)bh * J + j) * GA * U + u0, S_s, U, tid);
    __syncthreads();
    chunk_scalars(g_s, gam_s, a_s, b_s, tid);
    __syncthreads();

    {  // L and P
      float kk[4][4], qk[4][4];
      zero(kk); zero(qk);
      mm<4, 4, false, false>(kk, k_s, LDA_, k_s, LDA_, GA, ty, tx);
      mm<4, 4, false, false>(qk, q_s, LDA_, k_s, LDA_, GA, ty, tx);
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int d = 0; d < 4; ++d) {
          const int i = mi(c, ty), jj = ni<false>(d, tx);
          const float D = (i >= jj) ? expf(gam_s[i] - gam_s[jj]) : 0.f;
          L_s[i * LDC_ + jj] = (i > jj) ? beta_s[i] * kk[c][d] * D : 0.f;
          P_s[i * LDC_ + jj] = qk[c][d] * D;
        }
    }
    {  // r = beta (v - a (k S))
      float w[4][TNU];
      zero(w);
      mm<4, TNU, false, true>(w, k_s, LDA_, S_s, LDU, GA, ty, tx);
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int d = 0; d < TNU; ++d) {
          const int i = mi(c, ty), u = ni<true>(d, tx);
          n_s[i * LDU + u] = beta_s[i] * (n_s[i * LDU + u] - a_s[i] * w[c][d]);
        }
    }
    __syncthreads();
    if (tid < UB) {  // forward substitution, one column per thread
      float x[GC];
#pragma unroll
      for (int i = 0; i < GC; ++i) {
        float s = n_s[i * LDU + tid];
#pragma unroll
        for (int q4 = 0; q4 < (i + 3) / 4; ++q4) {
          const float4 l = *reinterpret_cast<const float4*>(L_s + i * LDC_ + 4 * q4);
          if (4 * q4 + 0 < i) s = fmaf(-l.x, x[4 * q4 + 0], s);
          if (4 * q4 + 1 < i) s = fmaf(-l.y, x[4 * q4 + 1], s);
          if (4 * q4 + 2 < i) s = fmaf(-l.z, x[4 * q4 + 2], s);
          if (4 * q4 + 3 < i) s = fmaf(-l.w, x[4 * q4 + 3], s);
        }
        x[i] = s;
      }
      float* no = p.n_out ? p.n_out + (row0 * p.H + h) * U + u0 + tid : nullptr;
#pragma unroll
      for (int i = 0; i < GC; ++i) {
        n_s[i * LDU + tid] = x[i];
        if (no) no[(long long)i * v_stride] = x[i];
      }
    }
    __syncthreads();
    {  // o = a (q S) + P n
      float o[4][TNU];
      zero(o);
      mm<4, TNU, false, true>(o, q_s, LDA_, S_s, LDU, GA, ty, tx);
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int d = 0; d < TNU; ++d) o[c][d] *= a_s[mi(c, ty)];
      mm<4, TNU, false, true>(o, P_s, LDC_, n_s, LDU, GC, ty, tx);
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int gq = 0; gq < TNU / 4; ++gq) {
          float* dst = p.o + ((row0 + mi(c, ty)) * p.H + h) * U + u0 + 64 * gq + 4 * tx;
          *reinterpret_cast<float4*>(dst) = make_float4(o[c][4 * gq], o[c][4 * gq + 1], o[c][4 * gq + 2], o[c][4 * gq + 3]);
        }
    }
    __syncthreads();  // every read of S is done
    {  // S' = a_C S + sum_j b_j k_j n_j^T
      float su[8][TNU];
      zero(su);
      mm<8, TNU, true, true>(su, k_s, LDA_, n_s, LDU, GC, ty, tx, b_s);
      const float aC = a_s[GC - 1];
#pragma unroll
      for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int d = 0; d < TNU; ++d) {
          float* s = S_s + mi(c, ty) * LDU + ni<true>(d, tx);
          *s = fmaf(aC, *s, su[c][d]);
        }
    }
    __syncthreads();
  }
  if (p.s_final) store_state<UB>(p.s_final + (long long)bh * GA * U + u0, S_s, U, tid);
}

// ----------------------------------------------------------------------------- backward
// One CTA per (batch, head, 64-wide slice of U); chunks are visited last to first.
constexpr int BU = 64;
constexpr int BLDU = BU + 4;

__global__ void __launch_bounds__(256, 1) gdn_bwd_kernel(GdnArgs p) {
  constexpr int NS = GA / BU;
  extern __shared__ __align__(16) float gsm[];
  float* S_s = gsm;                      // [128][68] chunk-start state
  float* dS_s = S_s + GA * BLDU;         // [128][68] gradient of the chunk-end state
  float* k_s = dS_s + GA * BLDU;         // [64][132]
  float* q_s = k_s + GC * LDA_;          // [64][132]
  float* n_s = q_s + GC * LDA_;          // [64][68]
  float* do_s = n_s + GC * BLDU;         // [64][68]
  float* dr_s = do_s + GC * BLDU;        // [64][68]  dn -> dr
  float* M_s = dr_s + GC * BLDU;         // [64][68]  L^T for the solve, later sym(dKK)
  float* P_s = M_s + GC * LDC_;          // [64][68]  P, later dQK
  float* g_s = P_s + GC * LDC_;
  float* beta_s = g_s + GC;
  float* gam_s = beta_s + GC;
  float* a_s = gam_s + GC;
  float* b_s = a_s + GC;
  float* wsc_s = b_s + GC;               // -beta_i a_i
  float* dgam_s = wsc_s + GC;
  float* dbeta_s = dgam_s + GC;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int bh = blockIdx.x / NS, us = blockIdx.x % NS;
  const int b = bh / p.H, h = bh % p.H, hk = h / (p.H / p.Hk);
  const int u0 = us * BU, U = p.U, T = p.T, J = T / GC;
  const long long qk_stride = (long long)p.Hk * GA, v_stride = (long long)p.H * U;

  load_state<BU>(dS_s, p.d_sfinal ? p.d_sfinal + (long long)bh * GA * U + u0 : nullptr, U, tid);
  __syncthreads();

  for (int j = J - 1; j >= 0; --j) {
    const long long row0 = (long long)b * T + (long long)j * GC;
    load_rows128(k_s, p.k + (row0 * p.Hk + hk) * GA, qk_stride, tid);
    load_rows128(q_s, p.q + (row0 * p.Hk + hk) * GA, qk_stride, tid);
    load_rowsU<BU>(n_s, p.n_out + (row0 * p.H + h) * U + u0, v_stride, tid);
    load_rowsU<BU>(do_s, p.d_o + (row0 * p.H + h) * U + u0, v_stride, tid);
    load_state<BU>(S_s, p.states + ((long long)bh * J + j) * GA * U + u0, U, tid);
    if (tid < GC) {
      g_s[tid] = p.g[(row0 + tid) * p.H + h];
      beta_s[tid] = p.beta[(row0 + tid) * p.H + h];
      dgam_s[tid] = 0.f;
      dbeta_s[tid] = 0.f;
    }
    __syncthreads();
    chunk_scalars(g_s, gam_s, a_s, b_s, tid);
    __syncthreads();
    if (tid < GC) wsc_s[tid] = -beta_s[tid] * a_s[tid];

    // ---- phase 1: KD = (k k^T) D kept in registers, L^T and P in shared memory
    float KD[4][4];
    {
      float qk[4][4];
      zero(KD); zero(qk);
      mm<4, 4, false, false>(KD, k_s, LDA_, k_s, LDA_, GA, ty, tx);
      mm<4, 4, false, false>(qk, q_s, LDA_, k_s, LDA_, GA, ty, tx);
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int d = 0; d < 4; ++d) {
          const int i = mi(c, ty), jj = ni<false>(d, tx);
          const float D = (i >= jj) ? expf(gam_s[i] - gam_s[jj]) : 0.f;
          KD[c][d] = (i > jj) ? KD[c][d] * D : 0.f;
          M_s[jj * LDC_ + i] = beta_s[i] * KD[c][d];   // L_ij stored transposed
          P_s[i * LDC_ + jj] = qk[c][d] * D;
        }
    }
    __syncthreads();

    // ---- phase 2: dn = P^T do + b (k dS')
    {
      float t1[4][4], t2[4][4];
      zero(t1); zero(t2);
      mm<4, 4, true, true>(t1, P_s, LDC_, do_s, BLDU, GC, ty, tx);
      mm<4, 4, false, true>(t2, k_s, LDA_, dS_s, BLDU, GA, ty, tx);
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int d = 0; d < 4; ++d) {
          const int jj = mi(c, ty), u = ni<true>(d, tx);
          dr_s[jj * BLDU + u] = fmaf(b_s[jj], t2[c][d], t1[c][d]);
        }
    }
    __syncthreads();

    // ---- phase 3: (I + L)^T dr = dn by back substitution, one column per thread; dv = beta dr
    if (tid < BU) {
      float x[GC];
#pragma unroll
      for (int i = GC - 1; i >= 0; --i) {
        float s = dr_s[i * BLDU + tid];
#pragma unroll
        for (int q4 = (i + 1) / 4; q4 < GC / 4; ++q4) {
          const float4 l = *reinterpret_cast<const float4*>(M_s + i * LDC_ + 4 * q4);
          if (4 * q4 + 0 > i) s = fmaf(-l.x, x[4 * q4 + 0], s);
          if (4 * q4 + 1 > i) s = fmaf(-l.y, x[4 * q4 + 1], s);
          if (4 * q4 + 2 > i) s = fmaf(-l.z, x[4 * q4 + 2], s);
          if (4 * q4 + 3 > i) s = fmaf(-l.w, x[4 * q4 + 3], s);
        }
        x[i] = s;
      }
      float* dvp = p.dv + (row0 * p.H + h) * U + u0 + tid;
#pragma unroll
      for (int i = 0; i < GC; ++i) {
        dr_s[i * BLDU + tid] = x[i];
        dvp[(long long)i * v_stride] = beta_s[i] * x[i];
      }
    }
    __syncthreads();

    // ---- phase 4: dP = do n^T, dL = -dr n^T; decay / beta gradients; dQK -> P_s, sym(dKK) -> M_s
    {
      float dp[4][4], dl[4][4];
      zero(dp); zero(dl);
      mm<4, 4, false, false>(dp, do_s, BLDU, n_s, BLDU, BU, ty, tx);
      mm<4, 4, false, false>(dl, dr_s, BLDU, n_s, BLDU, BU, ty, tx);
      float colE[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = mi(c, ty);
        const float bi = beta_s[i];
        float rowE = 0.f, rowB = 0.f;
#pragma unroll
        for (int d = 0; d < 4; ++d) {
          const int jj = ni<false>(d, tx);
          const float D = (i >= jj) ? expf(gam_s[i] - gam_s[jj]) : 0.f;
          const float dL = -dl[c][d];
          const float Pij = P_s[i * LDC_ + jj];
          P_s[i * LDC_ + jj] = dp[c][d] * D;                 // dQK (zero above the diagonal)
          float E = 0.f;
          if (i > jj) {
            rowB = fmaf(dL, KD[c][d], rowB);
            E = dL * bi * KD[c][d] + dp[c][d] * Pij;
            const float dKK = dL * bi * D;
            M_s[i * LDC_ + jj] = dKK;
            M_s[jj * LDC_ + i] = dKK;
          } else if (i == jj) {
            M_s[i * LDC_ + jj] = 0.f;
          }
          rowE += E;
          colE[d] += E;
        }
        rowE = half_warp_sum(rowE);
        rowB = half_warp_sum(rowB);
        if (tx == 0) {
          atomicAdd(dgam_s + i, rowE);
          atomicAdd(dbeta_s + i, rowB);
        }
      }
#pragma unroll
      for (int d = 0; d < 4; ++d) atomicAdd(dgam_s + ni<false>(d, tx), -colE[d]);
    }
    __syncthreads();

    // ---- phase 5: dbeta from r = beta (v - a W) with W = k S recomputed
    {
      float w[4][4];
      zero(w);
      mm<4, 4, false, true>(w, k_s, LDA_, S_s, BLDU, GA, ty, tx);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = mi(c, ty);
        const float4 vv = *reinterpret_cast<const float4*>(p.v + ((row0 + i) * p.H + h) * U + u0 + 4 * tx);
        const float4 dr = *reinterpret_cast<const float4*>(dr_s + i * BLDU + 4 * tx);
        const float ai = a_s[i];
        float s = dr.x * (vv.x - ai * w[c][0]) + dr.y * (vv.y - ai * w[c][1]) + dr.z * (vv.z - ai * w[c][2]) +
                  dr.w * (vv.w - ai * w[c][3]);
        s = half_warp_sum(s);
        if (tx == 0) atomicAdd(dbeta_s + i, s);
      }
    }

    // ---- phase 6: dq^T[a, i] = a_i sum_u S[a,u] do[i,u] + sum_j k[j,a] dQK[i,j]
    {
      float t[8][4];
      zero(t);
      mm<8, 4, false, false>(t, S_s, BLDU, do_s, BLDU, BU, ty, tx);
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        const int i = ni<false>(d, tx);
        const float ai = a_s[i];
        float dot = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          t[c][d] *= ai;
          dot = fmaf(q_s[i * LDA_ + mi(c, ty)], t[c][d], dot);   // d gamma_i += a_i do_i . (q S)_i
        }
        atomicAdd(dgam_s + i, dot);
      }
      mm<8, 4, true, false>(t, k_s, LDA_, P_s, LDC_, GC, ty, tx);
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        float* dst = p.dq + ((row0 + ni<false>(d, tx)) * p.Hk + hk) * GA;
        red_add_v4(dst + 4 * ty, t[0][d], t[1][d], t[2][d], t[3][d]);
        red_add_v4(dst + 64 + 4 * ty, t[4][d], t[5][d], t[6][d], t[7][d]);
      }
    }

    // ---- phase 7: dk^T[a, i] = -beta_i a_i sum_u S[a,u] dr[i,u] + b_i sum_u dS'[a,u] n[i,u]
    //                           + sum_j k[j,a] sym(dKK)[i,j]
    {
      float t[8][4], t2[8][4];
      zero(t); zero(t2);
      mm<8, 4, false, false>(t, S_s, BLDU, dr_s, BLDU, BU, ty, tx);
      mm<8, 4, false, false>(t2, dS_s, BLDU, n_s, BLDU, BU, ty, tx);
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        const int i = ni<false>(d, tx);
        const float ws = wsc_s[i], bi = b_s[i];
        float dot1 = 0.f, dot2 = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float kv = k_s[i * LDA_ + mi(c, ty)];
          const float x1 = ws * t[c][d];        // S-term of dk
          const float x2 = bi * t2[c][d];       // b-term of dk
          dot1 = fmaf(kv, x1, dot1);            // d gamma_i += dW_i . W_i
          dot2 = fmaf(kv, x2, dot2);            // b_i db_i
          t[c][d] = x1 + x2;
        }
        atomicAdd(dgam_s + i, dot1 - dot2);
        atomicAdd(dgam_s + GC - 1, dot2);
      }
      mm<8, 4, true, false>(t, k_s, LDA_, M_s, LDC_, GC, ty, tx);
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        float* dst = p.dk + ((row0 + ni<false>(d, tx)) * p.Hk + hk) * GA;
        red_add_v4(dst + 4 * ty, t[0][d], t[1][d], t[2][d], t[3][d]);
        red_add_v4(dst + 64 + 4 * ty, t[4][d], t[5][d], t[6][d], t[7][d]);
      }
    }
    {  // dk[j, a] += sum_i dQK[i,j] q[i,a]
      float t[4][8];
      zero(t);
      mm<4, 8, true, true>(t, P_s, LDC_, q_s, LDA_, GC, ty, tx);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float* dst = p.dk + ((row0 + mi(c, ty)) * p.Hk + hk) * GA;
        red_add_v4(dst + 4 * tx, t[c][0], t[c][1], t[c][2], t[c][3]);
        red_add_v4(dst + 64 + 4 * tx, t[c][4], t[c][5], t[c][6], t[c][7]);
      }
    }
    __syncthreads();  // every read of dS' is done

    // ---- phase 8: dS = a_C dS' + sum_i a_i q_i do_i^T + sum_i k_i dW_i^T, dW_i = -beta_i a_i dr_i
    {
      float t[8][4];
      zero(t);
      mm<8, 4, true, true>(t, q_s, LDA_, do_s, BLDU, GC, ty, tx, a_s);
      mm<8, 4, true, true>(t, k_s, LDA_, dr_s, BLDU, GC, ty, tx, wsc_s);
      const float aC = a_s[GC - 1];
      float part = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int d = 0; d < 4; ++d) {
          const int off = mi(c, ty) * BLDU + ni<true>(d, tx);
          const float old = dS_s[off];
          part = fmaf(S_s[off], old, part);
          dS_s[off] = fmaf(aC, old, t[c][d]);
        }
      part = warp_sum(part);
      if ((tid & 31) == 0) atomicAdd(dgam_s + GC - 1, aC * part);   // d gamma_C += a_C <S, dS'>
    }
    __syncthreads();

    // ---- phase 9: dg_t = sum_{i >= t} d gamma_i; partial over this U slice
    if (tid < GC) {
      float s = 0.f;
      for (int i = tid; i < GC; ++i) s += dgam_s[i];
      atomicAdd(p.dg + (row0 + tid) * p.H + h, s);
      atomicAdd(p.dbeta + (row0 + tid) * p.H + h, dbeta_s[tid]);
    }
    __syncthreads();
  }
  if (p.ds0) store_state<BU>(p.ds0 + (long long)bh * GA * U + u0, dS_s, U, tid);
}

}  // namespace ob

using namespace ob;

namespace {
template <int UB>
constexpr size_t fwd_smem() {
  return sizeof(float) * (size_t)(GA * (UB + 4) + 2 * GC * LDA_ + GC * (UB + 4) + 2 * GC * LDC_ + 5 * GC);
}
constexpr size_t bwd_smem() {
  return sizeof(float) * (size_t)(2 * GA * BLDU + 2 * GC * LDA_ + 3 * GC * BLDU + 2 * GC * LDC_ + 8 * GC);
}
int check_shape(int B, int T, int H, int Hk, int A, int U) {
  if (A != GA) return 6101;
  if (U % 64 || U <= 0) return 6102;
  if (T % GC || T <= 0) return 6103;
  if (Hk <= 0 || H % Hk) return 6104;
  if (B <= 0) return 6105;
  return 0;
}
}  // namespace

extern "C" {

// q,k [B,T,Hk,128] fp32; v [B,T,H,U]; g,beta [B,T,H]; s0/s_final [B,H,128,U] optional;
// n_out [B,T,H,U] and states [B,H,T/64,128,U] optional (needed by the backward).
int ob_gdn_fwd(const float* q, const float* k, const float* v, const float* g, const float* beta, const float* s0,
               float* o, float* n_out, float* states, float* s_final, int B, int T, int H, int Hk, int A, int U,
               cudaStream_t stream) {
  if (int e = check_shape(B, T, H, Hk, A, U)) return e;
  GdnArgs p{};
  p.q = q; p.k = k; p.v = v; p.g = g; p.beta = beta; p.s0 = s0;
  p.o = o; p.n_out = n_out; p.states = states; p.s_final = s_final;
  p.B = B; p.T = T; p.H = H; p.Hk = Hk; p.U = U;
  const bool wide = (U % 128 == 0) && ((long long)B * H * (U / 128) >= (num_sms() * 3) / 4);
  if (wide) {
    static bool attr = false;
    if (!attr) {
      cudaFuncSetAttribute(gdn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fwd_smem<128>());
      attr = true;
    }
    gdn_fwd_kernel<128><<<B * H * (U / 128), 256, fwd_smem<128>(), stream>>>(p);
  } else {
    static bool attr = false;
    if (!attr) {
      cudaFuncSetAttribute(gdn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fwd_smem<64>());
      attr = true;
    }
    gdn_fwd_kernel<64><<<B * H * (U / 64), 256, fwd_smem<64>(), stream>>>(p);
  }
  OB_CHECK_LAUNCH();
  return 0;
}

// dq, dk, dg, dbeta are accumulated into: the caller zero-fills them.
int ob_gdn_bwd(const float* q, const float* k, const float* v, const float* g, const float* beta,
               const float* n_out, const float* states, const float* d_o, const float* d_sfinal, float* dq,
               float* dk, float* dv, float* dg, float* dbeta, float* ds0, int B, int T, int H, int Hk, int A, int U,
               cudaStream_t stream) {
  if (int e = check_shape(B, T, H, Hk, A, U)) return e;
  GdnArgs p{};
  p.q = q; p.k = k; p.v = v; p.g = g; p.beta = beta;
  p.n_out = const_cast<float*>(n_out); p.states = const_cast<float*>(states);
  p.d_o = d_o; p.d_sfinal = d_sfinal;
  p.dq = dq; p.dk = dk; p.dv = dv; p.dg = dg; p.dbeta = dbeta; p.ds0 = ds0;
  p.B = B; p.T = T; p.H = H; p.Hk = Hk; p.U = U;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gdn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bwd_smem());
    attr = true;
  }
  gdn_bwd_kernel<<<B * H * (U / BU), 256, bwd_smem(), stream>>>(p);
  OB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
