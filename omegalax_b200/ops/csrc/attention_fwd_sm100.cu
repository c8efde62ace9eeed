// K3 forward: GQA flash attention for sm_100a on tcgen05 / TMEM.
//
// One CTA owns 256 consecutive query rows of one (sequence, query head): two 128-row
// tiles handled by two softmax warpgroups that ping-pong on the tensor core.
//   warp 0      TMA producer (Q once, then a 2-stage ring of K tiles and of V tiles)
//   warp 1      TMEM owner and the single tcgen05.mma issuing thread
//   warps 4-7   softmax warpgroup 0 (thread r <-> query row r, TMEM lane r)
//   warps 8-11  softmax warpgroup 1
// Per KV tile j and warpgroup w:  S_w = Q_w K_j^T lands in TMEM; the warpgroup reads its
// row, applies scale / mask / online softmax and writes P_w as packed bf16 back into the
// first half of the S_w columns; the issuing thread then runs O_w += P_w V_j with P_w as
// the TMEM A operand and V_j as an MN-major shared-memory B operand.  O_w stays in TMEM for
// the whole walk: the exponentials are taken against a reference maximum that is only moved
// (and O_w rescaled, a TMEM load / multiply / store by the warp that owns the rows) when a
// row's running maximum has grown by more than 2^8 since the reference was set, so in the
// common case a KV tile costs the warpgroup no accumulator traffic at all and it never waits
// for P V.  While warpgroup 0 does softmax, the tensor core works for warpgroup 1 and vice versa.
//
// Sequences are packed: row r of sequence b is global row cu_seqlens[b] + r.  Q/O are
// [rows, H, HD]; K/V are [rows, G, HD] with arbitrary row pitch (they may be slices of a
// fused QKV buffer).  LSE is written as [H, rows] in natural-log units for the backward.
#include "host_utils.h"
#include "sm100_common.cuh"

namespace ob {

constexpr int kAttnThreads = 384;

struct AttnFwdArgs {
  const int* cu_seqlens;  // [B+1]
  bf16* out;              // [rows, H, HD]
  long long o_row_stride;
  float* lse;             // [H, total_rows]
  long long total_rows;
  int H, G;
  int causal;
  float scale_log2;       // softmax scale * log2(e)
  int* status;
};

template <int HD>
struct AttnFwdSmem {
  static constexpr int kTile = 128 * HD * 2;          // one 128-row operand tile
  static constexpr int kQOff = 0;                     // 2 tiles
  static constexpr int kKOff = 2 * kTile;             // 2 stages
  static constexpr int kVOff = 4 * kTile;             // 2 stages
  static constexpr int kBarOff = 6 * kTile;
  static constexpr int kTotal = kBarOff + 256 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnFwdArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  using L = AttnFwdSmem<HD>;
  uint64_t* q_full = (uint64_t*)(smem + L::kBarOff);  // [2]
  uint64_t* k_full = q_full + 2;                      // [2]
  uint64_t* v_full = k_full + 2;                      // [2]
  uint64_t* k_empty = v_full + 2;                     // [2]
  uint64_t* v_empty = k_empty + 2;                    // [2]
  uint64_t* s_full = v_empty + 2;                     // [2]
  uint64_t* p_ready = s_full + 2;                     // [2]
  uint64_t* o_full = p_ready + 2;                     // [2]
  uint32_t* tmem_slot = (uint32_t*)(o_full + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int g = h / (p.H / p.G);
  const int seq_start = __ldg(p.cu_seqlens + b);
  const int seqlen = __ldg(p.cu_seqlens + b + 1) - seq_start;
  // heaviest (latest) query blocks first so the causal tail does not dominate
  const int qblk = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int q0 = qblk * 256;
  if (q0 >= seqlen) return;  // uniform for the whole CTA, nothing allocated yet

  const int n_kv_total = (seqlen + 127) >> 7;
  int n_w[2];
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    const int qs = q0 + w * 128;
    if (qs >= seqlen) n_w[w] = 0;
    else n_w[w] = p.causal ? min(n_kv_total, (qs >> 7) + 1) : n_kv_total;
  }
  const int n = max(n_w[0], n_w[1]);

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);
      mbar_init(&o_full[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+HD) O1 [384,384+HD)

  if (warp < 4) {
    setmaxnreg_dec<40>();
    if (warp == 0 && lane == 0) {
      // -------------------------------------------------------- TMA producer
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        if (n_w[w] > 0) {
          mbar_expect_tx(&q_full[w], L::kTile);
#pragma unroll
          for (int kb = 0; kb < HD / 64; ++kb)
            tma_load_3d(smem + L::kQOff + w * L::kTile + kb * 16384, &tmQ, &q_full[w], kb * 64, h,
                        seq_start + q0 + w * 128);
        }
      }
      bool ok = true;
      for (int j = 0; j < n && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        ok = mbar_wait(&k_empty[s], ph, abort_flag, p.status, OB_ERR_WAIT_EMPTY);
        if (!ok) break;
        mbar_expect_tx(&k_full[s], L::kTile);
#pragma unroll
        for (int kb = 0; kb < HD / 64; ++kb)
          tma_load_3d(smem + L::kKOff + s * L::kTile + kb * 16384, &tmK, &k_full[s], kb * 64, g,
                      seq_start + j * 128);
        ok = mbar_wait(&v_empty[s], ph, abort_flag, p.status, OB_ERR_WAIT_EMPTY);
        if (!ok) break;
        mbar_expect_tx(&v_full[s], L::kTile);
#pragma unroll
        for (int kb = 0; kb < HD / 64; ++kb)
          tma_load_3d(smem + L::kVOff + s * L::kTile + kb * 16384, &tmV, &v_full[s], kb * 64, g,
                      seq_start + j * 128);
      }
    } else if (warp == 1 && lane == 0) {
      // -------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, HD, 0, 1);
      auto issue_s = [&](int w, int s) {
        const uint32_t qa = smem_u32(smem + L::kQOff + w * L::kTile);
        const uint32_t ka = smem_u32(smem + L::kKOff + s * L::kTile);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_ss(tmem_base + w * 128, make_smem_desc(qa + off, 16, 1024),
                  make_smem_desc(ka + off, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int w, int s, bool first) {
        const uint32_t va = smem_u32(smem + L::kVOff + s * L::kTile);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // 16 keys per step: A = 8 packed TMEM columns, B advances 16 rows of 128 bytes
          umma_ts(tmem_base + 256 + w * 128, tmem_base + w * 128 + k * 8,
                  make_smem_desc(va + k * 2048, 16384, 1024), idesc_o, (!first || k > 0) ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(&k_full[0], 0, abort_flag, p.status, OB_ERR_WAIT_FULL);
      for (int w = 0; w < 2 && ok; ++w) {
        if (n_w[w] > 0) {
          ok = mbar_wait(&q_full[w], 0, abort_flag, p.status, OB_ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          issue_s(w, 0);
          umma_commit(&s_full[w]);
        }
      }
      if (ok) umma_commit(&k_empty[0]);
      for (int j = 0; j < n && ok; ++j) {
        const int s = j & 1;
        ok = mbar_wait(&v_full[s], (j >> 1) & 1, abort_flag, p.status, OB_ERR_WAIT_FULL);
        if (!ok) break;
        bool k_next_ready = false;
        for (int w = 0; w < 2 && ok; ++w) {
          if (j >= n_w[w]) continue;
          ok = mbar_wait(&p_ready[w], j & 1, abort_flag, p.status, OB_ERR_WAIT_MISC);
          if (!ok) break;
          tc_fence_after();
          issue_pv(w, s, j == 0);
          umma_commit(&o_full[w]);
          if (j + 1 < n_w[w]) {
            if (!k_next_ready) {
              ok = mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag, p.status,
                             OB_ERR_WAIT_FULL);
              if (!ok) break;
              tc_fence_after();
              k_next_ready = true;
            }
            issue_s(w, (j + 1) & 1);
            umma_commit(&s_full[w]);
          }
        }
        if (!ok) break;
        umma_commit(&v_empty[s]);
        if (j + 1 < n) umma_commit(&k_empty[(j + 1) & 1]);
      }
    }
  } else {
    setmaxnreg_inc<232>();
    // ---------------------------------------------------------- softmax warpgroups
    const int w = (warp >> 2) - 1;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                 // row inside the 128-row tile
    const int qpos = q0 + w * 128 + r;              // position inside the sequence
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_addr + w * 128;
    const uint32_t o_addr = tmem_base + lane_addr + 256 + w * 128;
    // m_ref: the maximum the exponentials (and O in TMEM) are currently taken against; m_run: the true
    // running maximum.  They differ by at most kRescaleLog2 between rescales.
    constexpr float kRescaleLog2 = 8.f;
    float m_ref = -INFINITY, m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    const int nj = n_w[w];
    for (int j = 0; j < nj && ok; ++j) {
      ok = mbar_wait(&s_full[w], j & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const int kbase = j * 128;
      const bool need_mask = (kbase + 128 > seqlen) || (p.causal && kbase + 127 > q0 + w * 128);
      const int klimit = p.causal ? min(seqlen - 1, qpos) : seqlen - 1;  // last visible key
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(s_addr + c * 32, v);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (kbase + c * 32 + i <= klimit) mx = fmaxf(mx, __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(v[i]));
        }
      }
      m_run = fmaxf(m_run, mx * p.scale_log2);
      // move the reference (and rescale O) only when some row of this warp needs it; the TMEM
      // accesses below are warp-wide, so the decision is too
      const bool mine = (m_run > m_ref + kRescaleLog2) || (m_ref == -INFINITY && m_run != -INFINITY);
      if (__any_sync(0xffffffffu, mine)) {
        const float m_new = mine ? m_run : m_ref;
        const float alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);   // 1 for rows that keep their reference
        if (j > 0) {   // O holds the products of the previous tiles: wait for the last of them, then rescale
          ok = mbar_wait(&o_full[w], (j - 1) & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL);
          if (!ok) break;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t v[32];
            tmem_ld32(o_addr + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st32(o_addr + c * 32, v);
          }
          tmem_st_wait();
        }
        l_run *= alpha;
        m_ref = m_new;
      }
      const float m_safe = (m_ref == -INFINITY) ? 0.f : m_ref;
      float lsum = 0.f;
      // pass 2: probabilities, packed bf16 into the first 64 columns of S
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(s_addr + c * 32, v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = fast_exp2(__uint_as_float(v[2 * i]) * p.scale_log2 - m_safe);
          float p1 = fast_exp2(__uint_as_float(v[2 * i + 1]) * p.scale_log2 - m_safe);
          if (need_mask) {
            if (kbase + c * 32 + 2 * i > klimit) p0 = 0.f;
            if (kbase + c * 32 + 2 * i + 1 > klimit) p1 = 0.f;
          }
          lsum += p0 + p1;
          pk[i] = pack_bf16(p0, p1);
        }
        tmem_st16(s_addr + c * 16, pk);
      }
      tmem_st_wait();
      l_run += lsum;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[w]);
    }
    // the accumulator of the last tile
    float o_acc[HD];
    if (ok && nj > 0) {
      ok = mbar_wait(&o_full[w], (nj - 1) & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(o_addr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = __uint_as_float(v[i]);
        }
        tc_fence_before();
      }
    }
    if (ok && nj > 0 && qpos < seqlen) {
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      const long long grow = (long long)seq_start + qpos;
      bf16* op = p.out + grow * p.o_row_stride + (long long)h * HD;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        uint4 q;
        q.x = pack_bf16(o_acc[i * 8 + 0] * inv_l, o_acc[i * 8 + 1] * inv_l);
        q.y = pack_bf16(o_acc[i * 8 + 2] * inv_l, o_acc[i * 8 + 3] * inv_l);
        q.z = pack_bf16(o_acc[i * 8 + 4] * inv_l, o_acc[i * 8 + 5] * inv_l);
        q.w = pack_bf16(o_acc[i * 8 + 6] * inv_l, o_acc[i * 8 + 7] * inv_l);
        *reinterpret_cast<uint4*>(op + i * 8) = q;
      }
      if (p.lse)   // l_run is relative to the reference maximum
        p.lse[(long long)h * p.total_rows + grow] =
            m_ref * 0.6931471805599453f + logf(fmaxf(l_run, 1e-30f));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    long long t0 = clock64();
    while (clock64() - t0 < 2000000) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HD>
static int launch_attn_fwd(const void* q, const void* k, const void* v, const AttnFwdArgs& a,
                           long long q_row_stride, long long k_row_stride, long long v_row_stride,
                           int B, int max_seqlen, cudaStream_t stream) {
  CUtensorMap tmQ, tmK, tmV;
  int e = make_tmap_3d(&tmQ, q, HD, a.H, a.total_rows, (uint64_t)HD * 2, (uint64_t)q_row_stride * 2,
                       64, 1, 128);
  if (e) return 2000 + e;
  e = make_tmap_3d(&tmK, k, HD, a.G, a.total_rows, (uint64_t)HD * 2, (uint64_t)k_row_stride * 2, 64,
                   1, 128);
  if (e) return 3000 + e;
  e = make_tmap_3d(&tmV, v, HD, a.G, a.total_rows, (uint64_t)HD * 2, (uint64_t)v_row_stride * 2, 64,
                   1, 128);
  if (e) return 3500 + e;
  auto kern = attn_fwd_kernel<HD>;
  OB_ENSURE_DYN_SMEM(kern, AttnFwdSmem<HD>::kTotal);
  dim3 grid((max_seqlen + 255) / 256, a.H, B);
  kern<<<grid, kAttnThreads, AttnFwdSmem<HD>::kTotal, stream>>>(tmQ, tmK, tmV, a);
  OB_CHECK_LAUNCH();
  return 0;
}

// attention_fwd256_sm100.cu
int launch_attn_fwd256(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_seqlens, int B,
                       int max_seqlen, long long total_rows, int H, int G, long long q_row_stride,
                       long long k_row_stride, long long v_row_stride, long long o_row_stride, float scale, int causal,
                       int* status, cudaStream_t stream);

}  // namespace ob

using namespace ob;

extern "C" {

// q/out: [total_rows, H, HD]; k, v: [total_rows, G, HD]; row strides in elements.
// cu_seqlens: device int32 [B+1].  lse: [H, total_rows] fp32 (may be null).
int ob_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                const int* cu_seqlens, int B, int max_seqlen, long long total_rows, int H, int G,
                int HD, long long q_row_stride, long long k_row_stride, long long v_row_stride,
                long long o_row_stride, float scale, int causal, int* status,
                cudaStream_t stream) {
  if (B <= 0 || total_rows <= 0) return 0;
  if ((q_row_stride & 7) || (k_row_stride & 7) || (v_row_stride & 7) || (o_row_stride & 7))
    return 6001;
  if ((((uintptr_t)q) | ((uintptr_t)k) | ((uintptr_t)v) | ((uintptr_t)out)) & 15) return 6002;
  AttnFwdArgs a = {};
  a.cu_seqlens = cu_seqlens;
  a.out = (bf16*)out;
  a.o_row_stride = o_row_stride;
  a.lse = lse;
  a.total_rows = total_rows;
  a.H = H; a.G = G; a.causal = causal;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  if (HD == 128)
    return launch_attn_fwd<128>(q, k, v, a, q_row_stride, k_row_stride, v_row_stride, B, max_seqlen,
                                stream);
  if (HD == 64)
    return launch_attn_fwd<64>(q, k, v, a, q_row_stride, k_row_stride, v_row_stride, B, max_seqlen,
                               stream);
  if (HD == 256)
    return launch_attn_fwd256(q, k, v, out, lse, cu_seqlens, B, max_seqlen, total_rows, H, G, q_row_stride,
                              k_row_stride, v_row_stride, o_row_stride, scale, causal, status, stream);
  return 6005;
}

}  // extern "C"
