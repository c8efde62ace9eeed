// K3 forward for 256-wide heads (Qwen3.5 gated attention: 32 query / 2 kv heads of 256).
//
// One CTA owns 128 consecutive query rows of one (sequence, query head).  The 128 x 256 fp32 output
// does not fit one thread's registers, so two warpgroups share the tile by head-dim halves:
//   warp 0      TMA producer (Q once, then one K tile and one V tile in flight: 3 x 64 KB of
//               shared memory hold Q, K_j and V_j)
//   warp 1      TMEM owner and the single tcgen05.mma issuing thread
//   warps 4-7   warpgroup 0: online softmax of S (thread r <-> query row r), writes P as packed
//               bf16 into TMEM and the per-row rescale factor into shared memory, accumulates
//               O[:, 0:128] in registers
//   warps 8-11  warpgroup 1: accumulates O[:, 128:256] in registers with the same factors
// Per KV tile j:  S = Q K_j^T (16 k-steps over the 256 head dims) lands in TMEM columns [0,128);
// warpgroup 0 turns it into P (first 64 columns); O_j = P V_j (A from TMEM, B = V_j as an MN-major
// tile, N = 256) lands in columns [128,384) and both warpgroups fold their half into their
// accumulators.  K_{j+1} streams in while softmax and P V of tile j run (its buffer is free once
// S_j is complete), V_{j+1} while S_{j+1} and its softmax run.
//
// Layout of the tensors, sequence packing and the LSE output are those of attention_fwd_sm100.cu.
#include "host_utils.h"
#include "sm100_common.cuh"

namespace ob {

constexpr int kF256Threads = 384;
constexpr int kF256HD = 256;

struct AttnFwd256Args {
  const int* cu_seqlens;
  bf16* out;
  long long o_row_stride;
  float* lse;
  long long total_rows;
  int H, G;
  int causal;
  float scale_log2;
  int* status;
};

struct AttnFwd256Smem {
  static constexpr int kTile = 128 * kF256HD * 2;   // 64 KB: 4 boxes of 128 rows x 64 columns
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kTile;
  static constexpr int kVOff = 2 * kTile;
  static constexpr int kAlphaOff = 3 * kTile;       // 2 x 128 rescale factors, then 128 x 1/l
  static constexpr int kBarOff = kAlphaOff + 3 * 512;
  static constexpr int kTotal = kBarOff + 256 + 1024;
};

__global__ void __launch_bounds__(kF256Threads, 1)
attn_fwd256_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const AttnFwd256Args p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  using L = AttnFwd256Smem;
  uint64_t* q_full = (uint64_t*)(smem + L::kBarOff);
  uint64_t* k_full = q_full + 1;
  uint64_t* v_full = k_full + 1;
  uint64_t* k_empty = v_full + 1;
  uint64_t* v_empty = k_empty + 1;
  uint64_t* s_full = v_empty + 1;
  uint64_t* p_ready = s_full + 1;     // 4 warps of warpgroup 0
  uint64_t* o_full = p_ready + 1;
  uint64_t* o_read = o_full + 1;      // 8 warps: both warpgroups have folded the scratch accumulator
  uint32_t* tmem_slot = (uint32_t*)(o_read + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  float* alpha_s = reinterpret_cast<float*>(smem + L::kAlphaOff);   // [2][128]
  float* linv_s = alpha_s + 256;                                    // [128]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int g = h / (p.H / p.G);
  const int seq_start = __ldg(p.cu_seqlens + b);
  const int seqlen = __ldg(p.cu_seqlens + b + 1) - seq_start;
  const int qblk = (int)gridDim.x - 1 - (int)blockIdx.x;   // heaviest query blocks first
  const int q0 = qblk * 128;
  if (q0 >= seqlen) return;
  const int n_kv_total = (seqlen + 127) >> 7;
  const int n = p.causal ? min(n_kv_total, (q0 >> 7) + 1) : n_kv_total;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 4);
    mbar_init(o_full, 1);
    mbar_init(o_read, 8);
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
  const uint32_t T_S = tmem_base, T_O = tmem_base + 128;

  if (warp < 4) {
    setmaxnreg_dec<40>();
    if (warp == 0 && lane == 0) {
      // -------------------------------------------------------- TMA producer
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, L::kTile);
#pragma unroll
      for (int kb = 0; kb < kF256HD / 64; ++kb)
        tma_load_3d(smem + L::kQOff + kb * 16384, &tmQ, q_full, kb * 64, h, seq_start + q0);
      bool ok = true;
      for (int j = 0; j < n && ok; ++j) {
        const uint32_t ph = (j & 1) ^ 1;
        ok = mbar_wait(k_empty, ph, abort_flag, p.status, OB_ERR_WAIT_EMPTY);
        if (!ok) break;
        mbar_expect_tx(k_full, L::kTile);
#pragma unroll
        for (int kb = 0; kb < kF256HD / 64; ++kb)
          tma_load_3d(smem + L::kKOff + kb * 16384, &tmK, k_full, kb * 64, g, seq_start + j * 128);
        ok = mbar_wait(v_empty, ph, abort_flag, p.status, OB_ERR_WAIT_EMPTY);
        if (!ok) break;
        mbar_expect_tx(v_full, L::kTile);
#pragma unroll
        for (int kb = 0; kb < kF256HD / 64; ++kb)
          tma_load_3d(smem + L::kVOff + kb * 16384, &tmV, v_full, kb * 64, g, seq_start + j * 128);
      }
    } else if (warp == 1 && lane == 0) {
      // -------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, kF256HD, 0, 1);
      const uint32_t qa = smem_u32(smem + L::kQOff), ka = smem_u32(smem + L::kKOff), va = smem_u32(smem + L::kVOff);
      auto issue_s = [&]() {
#pragma unroll
        for (int k = 0; k < kF256HD / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_ss(T_S, make_smem_desc(qa + off, 16, 1024), make_smem_desc(ka + off, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, OB_ERR_WAIT_FULL);
      if (ok) ok = mbar_wait(k_full, 0, abort_flag, p.status, OB_ERR_WAIT_FULL);
      if (ok) {
        tc_fence_after();
        issue_s();
        umma_commit(s_full);
        umma_commit(k_empty);
      }
      for (int j = 0; j < n && ok; ++j) {
        ok = mbar_wait(p_ready, j & 1, abort_flag, p.status, OB_ERR_WAIT_MISC);
        if (ok) ok = mbar_wait(v_full, j & 1, abort_flag, p.status, OB_ERR_WAIT_FULL);
        if (ok && j > 0) ok = mbar_wait(o_read, (j - 1) & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)   // 16 keys per step: A = 8 packed TMEM columns, B advances 16 key rows
          umma_ts(T_O, T_S + k * 8, make_smem_desc(va + k * 2048, 16384, 1024), idesc_o, k > 0 ? 1u : 0u);
        umma_commit(o_full);
        umma_commit(v_empty);
        if (j + 1 < n) {
          ok = mbar_wait(k_full, (j + 1) & 1, abort_flag, p.status, OB_ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          issue_s();               // executes after P V of tile j, which read P from these columns
          umma_commit(s_full);
          umma_commit(k_empty);
        }
      }
    }
  } else {
    setmaxnreg_inc<232>();
    const int wg = (warp >> 2) - 1;                 // 0: softmax + O[:, :128], 1: O[:, 128:]
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int qpos = q0 + r;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const uint32_t s_addr = T_S + lane_addr;
    const uint32_t o_addr = T_O + lane_addr + wg * 128;
    float o_acc[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n && ok; ++j) {
      float alpha;
      if (wg == 0) {
        ok = mbar_wait(s_full, j & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        const int kbase = j * 128;
        const bool need_mask = (kbase + 128 > seqlen) || (p.causal && kbase + 127 > q0);
        const int klimit = p.causal ? min(seqlen - 1, qpos) : seqlen - 1;
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
        const float m_new = fmaxf(m_run, mx * p.scale_log2);
        const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
        alpha = fast_exp2(m_run - m_safe);
        m_run = m_new;
        float lsum = 0.f;
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
        l_run = l_run * alpha + lsum;
        alpha_s[(j & 1) * 128 + r] = alpha;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready);
      } else {
        ok = mbar_wait(p_ready, j & 1, abort_flag, p.status, OB_ERR_WAIT_MISC);   // the factors are in shared memory
        if (!ok) break;
        alpha = alpha_s[(j & 1) * 128 + r];
      }
      ok = mbar_wait(o_full, j & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(o_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + __uint_as_float(v[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_read);
    }
    // 1 / l travels from warpgroup 0 to warpgroup 1 through shared memory
    if (wg == 0) linv_s[r] = l_run > 0.f ? 1.f / l_run : 0.f;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (ok && qpos < seqlen) {
      const float inv_l = linv_s[r];
      const long long grow = (long long)seq_start + qpos;
      bf16* op = p.out + grow * p.o_row_stride + (long long)h * kF256HD + wg * 128;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        uint4 q;
        q.x = pack_bf16(o_acc[i * 8 + 0] * inv_l, o_acc[i * 8 + 1] * inv_l);
        q.y = pack_bf16(o_acc[i * 8 + 2] * inv_l, o_acc[i * 8 + 3] * inv_l);
        q.z = pack_bf16(o_acc[i * 8 + 4] * inv_l, o_acc[i * 8 + 5] * inv_l);
        q.w = pack_bf16(o_acc[i * 8 + 6] * inv_l, o_acc[i * 8 + 7] * inv_l);
        *reinterpret_cast<uint4*>(op + i * 8) = q;
      }
      if (wg == 0 && p.lse)
        p.lse[(long long)h * p.total_rows + grow] = m_run * 0.6931471805599453f + logf(fmaxf(l_run, 1e-30f));
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

// Called by ob_attn_fwd for HD == 256.
int launch_attn_fwd256(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_seqlens, int B,
                       int max_seqlen, long long total_rows, int H, int G, long long q_row_stride,
                       long long k_row_stride, long long v_row_stride, long long o_row_stride, float scale, int causal,
                       int* status, cudaStream_t stream) {
  CUtensorMap tmQ, tmK, tmV;
  int e = make_tmap_3d(&tmQ, q, kF256HD, H, total_rows, (uint64_t)kF256HD * 2, (uint64_t)q_row_stride * 2, 64, 1, 128);
  if (e) return 2000 + e;
  e = make_tmap_3d(&tmK, k, kF256HD, G, total_rows, (uint64_t)kF256HD * 2, (uint64_t)k_row_stride * 2, 64, 1, 128);
  if (e) return 3000 + e;
  e = make_tmap_3d(&tmV, v, kF256HD, G, total_rows, (uint64_t)kF256HD * 2, (uint64_t)v_row_stride * 2, 64, 1, 128);
  if (e) return 3500 + e;
  OB_ENSURE_DYN_SMEM(attn_fwd256_kernel, AttnFwd256Smem::kTotal);
  AttnFwd256Args a = {};
  a.cu_seqlens = cu_seqlens;
  a.out = (bf16*)out;
  a.o_row_stride = o_row_stride;
  a.lse = lse;
  a.total_rows = total_rows;
  a.H = H; a.G = G; a.causal = causal;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  dim3 grid((max_seqlen + 127) / 128, H, B);
  attn_fwd256_kernel<<<grid, kF256Threads, AttnFwd256Smem::kTotal, stream>>>(tmQ, tmK, tmV, a);
  OB_CHECK_LAUNCH();
  return 0;
}

}  // namespace ob
