// K3 backward: GQA flash attention gradients for sm_100a on tcgen05 / TMEM (head_dim 128).
//
// One CTA owns one 128-key tile of one (sequence, kv head) and walks over every query head
// of the group and every 64-query tile that can see those keys.  dK and dV accumulate in
// TMEM for the whole walk (no atomics); dQ is produced per step as a transposed tile and
// added into an fp32 accumulation buffer with coalesced red.global.add.
//
// Per step (64 queries), with everything "transposed" so that thread r <-> key row r:
//   A1  S^T  = K  Q^T          (M=128 keys, N=64 queries, reduce head_dim)      -> TMEM
//   A2  dP^T = V  dO^T                                                           -> TMEM
//   E   P^T = exp2(S^T*scale - lse), dS^T = P^T * (dP^T - delta) * scale   (threads)
//       P^T, dS^T  -> packed bf16 into TMEM (A operands); dS^T also -> shared memory
//   B1  dV  += P^T  dO         (A from TMEM, B = dO as MN-major tile)
//   B2  dK  += dS^T Q          (A from TMEM, B = Q  as MN-major tile)
//   B3  dQ^T = K^T dS          (A = K as MN-major tile, B = dS^T tile in shared memory)
//   D   dQ^T goes through a transposing shared-memory tile into the fp32 dQ buffer (TMA reduce-add)
// S^T/dP^T are double buffered so A(i+1) runs while the threads are in E(i); dQ^T(i)
// reuses the S^T buffer of step i.  Q/dO tiles come through a 3-stage TMA ring.
// E runs on eight warps (two per TMEM lane quadrant, 32 query columns each), D on four warps of
// its own (one per quadrant, 64 columns), so draining dQ^T of step i-1 overlaps E of step i and
// the S^T buffer is handed back to the tensor core without waiting for the softmax warps.
//
// Heads of 256 (template HD = 256): dK and dV of a 128-key tile would need all 512 TMEM columns, so
// the kernel runs twice, once per 128-wide half `dh` of the head dimension.  Each pass computes
// S^T and dP^T over all 256 dimensions (they need the full dot products) and the three gradient
// products for its half only (dV[:, half], dK[:, half], dQ[:, half]).  The K and V tiles take
// 128 KB of shared memory there, which leaves room for a single Q/dO stage and no dQ staging tile:
// the dQ warps add their dQ^T rows to the fp32 buffer with coalesced red.global.add instead.
//
// Scratch (allocated by the caller): delta [H, rows] fp32 = rowsum(dO * O) from the
// preprocess kernel, and dq_acc [rows, H, 128] fp32, zeroed before launch and converted to
// bf16 by the postprocess kernel.
#include "host_utils.h"
#include "sm100_common.cuh"

namespace ob {

constexpr int kBwdThreads = 448;     // producer warp, MMA warp, 8 softmax/dS warps, 4 dQ warps
constexpr int kHD = 128;       // width of the head-dim slice one pass produces gradients for
constexpr int kQT = 64;        // queries per step

struct AttnBwdArgs {
  const int* cu_seqlens;
  const float* lse;      // [H, rows] natural log
  const float* delta;    // [H, rows]
  float* dq_acc;         // [rows, H, 128] fp32
  bf16* dk;              // [rows, G, 128] with row stride
  bf16* dv;
  long long dk_row_stride, dv_row_stride;
  long long total_rows;
  int H, G;
  int causal;
  int dh;                // which 128-wide half of the head dimension this pass differentiates (HD 256)
  float scale, scale_log2;
  int* status;
};

template <int HD>
struct AttnBwdSmem {
  static constexpr int kStages = HD == 128 ? 3 : 1;     // Q/dO ring depth
  static constexpr int kKVTile = 128 * HD * 2;          // 32 KB (HD 128) / 64 KB (HD 256)
  static constexpr int kQTile = kQT * HD * 2;           // 16 KB / 32 KB
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kKVTile;
  static constexpr int kQOff = 2 * kKVTile;
  static constexpr int kDOOff = kQOff + kStages * kQTile;
  static constexpr int kDSOff = kDOOff + kStages * kQTile;  // 2 x 16 KB
  static constexpr int kDQOff = kDSOff + 2 * 16384;         // 32 KB fp32 [64 q][128 d] staging (HD 128 only)
  static constexpr int kStatOff = kDQOff + (HD == 128 ? 32768 : 0);   // per stage 64 lse*log2e + 64 delta, fp32
  static constexpr int kBarOff = kStatOff + kStages * 512;
  static constexpr int kTotal = kBarOff + 256 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                const __grid_constant__ CUtensorMap tmDQ, const AttnBwdArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  using L = AttnBwdSmem<HD>;
  constexpr int kQStages = L::kStages;
  uint64_t* kv_full = (uint64_t*)(smem + L::kBarOff);  // [1]
  uint64_t* qdo_full = kv_full + 1;                    // [3]
  uint64_t* qdo_empty = qdo_full + kQStages;           // [3]
  uint64_t* sp_full = qdo_empty + kQStages;            // [2]
  uint64_t* ds_ready = sp_full + 2;                    // [2]
  uint64_t* dq_full = ds_ready + 2;                    // [2]
  uint64_t* dq_read = dq_full + 2;                     // [2]
  uint64_t* dkv_full = dq_read + 2;                    // [1]
  uint64_t* dqs_free = dkv_full + 1;                   // [1] dQ staging tile may be overwritten
  uint64_t* dqs_full = dqs_free + 1;                   // [1] dQ staging tile fully written
  uint32_t* tmem_slot = (uint32_t*)(dqs_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int g = blockIdx.y;
  const int R = p.H / p.G;
  const int seq_start = __ldg(p.cu_seqlens + b);
  const int seqlen = __ldg(p.cu_seqlens + b + 1) - seq_start;
  const int k0 = blockIdx.x * 128;
  if (k0 >= seqlen) return;
  const int nq_total = (seqlen + kQT - 1) / kQT;
  const int i_first = p.causal ? (k0 / kQT) : 0;
  const int nqt = nq_total - i_first;   // query tiles per head (>= 1 because k0 < seqlen)
  const int n = R * nqt;                // steps of this CTA

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < kQStages; ++i) {
      mbar_init(&qdo_full[i], 2);  // TMA expect_tx arrival + row statistics arrival
      mbar_init(&qdo_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sp_full[i], 1);
      mbar_init(&ds_ready[i], 8);
      mbar_init(&dq_full[i], 1);
      mbar_init(&dq_read[i], 4);
    }
    mbar_init(dkv_full, 1);
    mbar_init(dqs_free, 1);
    mbar_init(dqs_full, 4);
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
  // TMEM columns: dK [0,128) dV [128,256) S^T {256,320} dP^T {384,448}
  const uint32_t T_DK = tmem_base, T_DV = tmem_base + 128;
  auto T_S = [&](int bb) { return tmem_base + 256 + bb * 64; };
  auto T_DP = [&](int bb) { return tmem_base + 384 + bb * 64; };

  if (warp == 0) {
    // ------------------------------------------------------------ producer warp
    // lane 0 drives the TMA ring; all 32 lanes stage the per-query statistics of the step
    // (lse * log2(e) and delta, 64 each) into shared memory next to the Q/dO tiles.
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmDO);
      mbar_expect_tx(kv_full, 2 * L::kKVTile);
      for (int kb = 0; kb < HD / 64; ++kb) {
        tma_load_3d(smem + L::kKOff + kb * 16384, &tmK, kv_full, kb * 64, g, seq_start + k0);
        tma_load_3d(smem + L::kVOff + kb * 16384, &tmV, kv_full, kb * 64, g, seq_start + k0);
      }
    }
    bool ok = true;
    for (int it = 0; it < n; ++it) {
      const int s = it % kQStages;
      const uint32_t ph = ((it / kQStages) & 1) ^ 1;
      if (lane == 0) ok = mbar_wait(&qdo_empty[s], ph, abort_flag, p.status, OB_ERR_WAIT_EMPTY);
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      if (!ok) break;
      const int h = g * R + it / nqt;
      const int q0 = (i_first + it % nqt) * kQT;
      if (lane == 0) {
        mbar_expect_tx(&qdo_full[s], 2 * L::kQTile);
        for (int kb = 0; kb < HD / 64; ++kb) {
          tma_load_3d(smem + L::kQOff + s * L::kQTile + kb * 8192, &tmQ, &qdo_full[s], kb * 64, h,
                      seq_start + q0);
          tma_load_3d(smem + L::kDOOff + s * L::kQTile + kb * 8192, &tmDO, &qdo_full[s], kb * 64, h,
                      seq_start + q0);
        }
      }
      float* st = reinterpret_cast<float*>(smem + L::kStatOff + s * 512);
      const int qvalid = min(kQT, seqlen - q0);
      const long long base = (long long)h * p.total_rows + seq_start + q0;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int qq = lane + 32 * j;
        const int qc = qq < qvalid ? qq : 0;
        st[qq] = __ldg(p.lse + base + qc) * 1.4426950408889634f;
        st[64 + qq] = __ldg(p.delta + base + qc);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&qdo_full[s]);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_a = make_idesc_bf16(128, kQT, 0, 0);   // S^T, dP^T
      constexpr uint32_t idesc_b = make_idesc_bf16(128, kHD, 0, 1);   // dV, dK (A in TMEM)
      constexpr uint32_t idesc_q = make_idesc_bf16(128, kQT, 1, 1);   // dQ^T
      const uint32_t ka = smem_u32(smem + L::kKOff), va = smem_u32(smem + L::kVOff);
      auto issue_A = [&](int it) {
        const int s = it % kQStages, bb = it & 1;
        const uint32_t qa = smem_u32(smem + L::kQOff + s * L::kQTile);
        const uint32_t da = smem_u32(smem + L::kDOOff + s * L::kQTile);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t offA = (k >> 2) * 16384 + (k & 3) * 32;
          const uint32_t offB = (k >> 2) * 8192 + (k & 3) * 32;
          umma_ss(T_S(bb), make_smem_desc(ka + offA, 16, 1024), make_smem_desc(qa + offB, 16, 1024),
                  idesc_a, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t offA = (k >> 2) * 16384 + (k & 3) * 32;
          const uint32_t offB = (k >> 2) * 8192 + (k & 3) * 32;
          umma_ss(T_DP(bb), make_smem_desc(va + offA, 16, 1024), make_smem_desc(da + offB, 16, 1024),
                  idesc_a, k > 0 ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, OB_ERR_WAIT_FULL);
      if (ok) ok = mbar_wait(&qdo_full[0], 0, abort_flag, p.status, OB_ERR_WAIT_FULL);
      if (ok) {
        tc_fence_after();
        issue_A(0);
        umma_commit(&sp_full[0]);
      }
      // A(it+1): S^T / dP^T of the next step.  With a Q/dO ring it is issued ahead of B(it) so that it
      // runs while the threads are in E(it); with a single stage (256-wide heads) its operands can
      // only be loaded once B(it) has released the stage, so it follows B(it).
      auto issue_next = [&](int it) -> bool {
        if (it + 1 >= n) return true;
        const int nx = it + 1;
        if (nx >= 2) {  // the S^T buffer of step nx still holds dQ^T of step nx-2
          if (!mbar_wait(&dq_read[nx & 1], ((nx - 2) >> 1) & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY))
            return false;
        }
        if (!mbar_wait(&qdo_full[nx % kQStages], (nx / kQStages) & 1, abort_flag, p.status, OB_ERR_WAIT_FULL))
          return false;
        tc_fence_after();
        issue_A(nx);
        umma_commit(&sp_full[nx & 1]);
        return true;
      };
      for (int it = 0; it < n && ok; ++it) {
        const int bb = it & 1;
        if (kQStages > 1) {
          ok = issue_next(it);
          if (!ok) break;
        }
        ok = mbar_wait(&ds_ready[bb], (it >> 1) & 1, abort_flag, p.status, OB_ERR_WAIT_MISC);
        if (!ok) break;
        tc_fence_after();
        const int s = it % kQStages;
        // the 128-wide head-dim slice of this pass: two 64-column blocks of every tile
        const uint32_t qa = smem_u32(smem + L::kQOff + s * L::kQTile) + p.dh * 16384;
        const uint32_t da = smem_u32(smem + L::kDOOff + s * L::kQTile) + p.dh * 16384;
        const uint32_t kah = ka + p.dh * 32768;
        const uint32_t dsa = smem_u32(smem + L::kDSOff + bb * 16384);
        // dV += P^T dO ; dK += dS^T Q : reduce over the 64 queries (4 steps of 16)
#pragma unroll
        for (int k = 0; k < kQT / 16; ++k)
          umma_ts(T_DV, T_S(bb) + (k >> 1) * 32 + (k & 1) * 8, make_smem_desc(da + k * 2048, 8192, 1024), idesc_b,
                  (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < kQT / 16; ++k)
          umma_ts(T_DK, T_DP(bb) + (k >> 1) * 32 + (k & 1) * 8, make_smem_desc(qa + k * 2048, 8192, 1024), idesc_b,
                  (it > 0 || k > 0) ? 1u : 0u);
        // dQ^T = K^T dS : reduce over the 128 keys (8 steps of 16)
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(T_S(bb), make_smem_desc(kah + k * 2048, 16384, 1024),
                  make_smem_desc(dsa + k * 2048, 16384, 1024), idesc_q, k > 0 ? 1u : 0u);
        umma_commit(&dq_full[bb]);
        umma_commit(&qdo_empty[s]);
        if (kQStages == 1) ok = issue_next(it);
      }
      if (ok) umma_commit(dkv_full);
    }
  } else if (warp >= 10) {
    // ------------------------------------------------------------ dQ warps (10..13)
    // D(it): move dQ^T of step `it` from TMEM through a transposing shared-memory tile into the
    // fp32 dQ buffer with one TMA reduce-add (no per-element atomics).  One warp per TMEM lane
    // quadrant; thread r holds head-dim index r of all 64 queries of the step.
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const bool issuer = (warp == 10 && lane == 0);
    float* dq_s = reinterpret_cast<float*>(smem + L::kDQOff);
    bool ok = true;
    for (int it = 0; it < n && ok; ++it) {
      const int bb = it & 1;
      ok = mbar_wait(&dq_full[bb], (it >> 1) & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL);
      __syncwarp();
      if (!ok) break;
      tc_fence_after();
      uint32_t v0[32], v1[32];
      tmem_ld32(T_S(bb) + lane_addr, v0);
      tmem_ld32(T_S(bb) + lane_addr + 32, v1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dq_read[bb]);   // the tensor core may overwrite this S^T buffer
      if constexpr (HD != 128) {
        // no staging tile: thread r adds head-dim element r of every query row (a warp covers 128
        // consecutive bytes of one row per instruction)
        const int h = g * R + it / nqt;
        const int q0 = (i_first + it % nqt) * kQT;
        const int qvalid = min(kQT, seqlen - q0);
        float* dst = p.dq_acc + ((long long)(seq_start + q0) * p.H + h) * HD + p.dh * kHD + r;
        const long long rs = (long long)p.H * HD;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i < qvalid) atomicAdd(dst + i * rs, __uint_as_float(v0[i]));
          if (32 + i < qvalid) atomicAdd(dst + (32 + i) * rs, __uint_as_float(v1[i]));
        }
        continue;
      }
      // the staging tile is free once the previous reduce-add has read it
      if (issuer) {
        tma_store_wait_read<0>();
        mbar_arrive(dqs_free);
      }
      ok = mbar_wait(dqs_free, it & 1, abort_flag, p.status, OB_ERR_WAIT_MISC);
      if (!ok) break;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        dq_s[i * kHD + r] = __uint_as_float(v0[i]);
        dq_s[(32 + i) * kHD + r] = __uint_as_float(v1[i]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(dqs_full);
      if (issuer) {
        ok = mbar_wait(dqs_full, it & 1, abort_flag, p.status, OB_ERR_WAIT_MISC);
        if (ok) {
          const int h = g * R + it / nqt;
          const int q0 = (i_first + it % nqt) * kQT;
          tma_reduce_add_2d(&tmDQ, dq_s, h * kHD, seq_start + q0);
          tma_store_commit();
        }
      }
    }
    if (issuer) tma_store_wait_all<0>();
  } else {
    // ------------------------------------------------------------ softmax / dS warps (2..9)
    // Two warps share each TMEM lane quadrant and split the 64 query columns of a step.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;          // which 32 query columns
    const int r = quad * 32 + lane;            // key row
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const int kpos = k0 + r;
    const bool key_ok = kpos < seqlen;
    bool ok = true;
    for (int it = 0; it < n && ok; ++it) {
      const int bb = it & 1;
      const int s = it % kQStages;
      ok = mbar_wait(&sp_full[bb], (it >> 1) & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL);
      // the statistics of this step were published on the stage barrier (already complete)
      if (ok) ok = mbar_wait(&qdo_full[s], (it / kQStages) & 1, abort_flag, p.status, OB_ERR_WAIT_FULL);
      __syncwarp();
      if (!ok) break;
      tc_fence_after();
      const int q0 = (i_first + it % nqt) * kQT;
      const int qvalid = min(kQT, seqlen - q0);
      const bool need_mask = (qvalid < kQT) || (k0 + 128 > seqlen) || (p.causal && q0 < k0 + 127);
      const float4* st_l = reinterpret_cast<const float4*>(smem + L::kStatOff + s * 512) + half * 8;
      const float4* st_d = st_l + 16;
      uint8_t* ds_row = smem + L::kDSOff + bb * 16384 + r * 128;
      uint32_t sv[32], dv[32];
      tmem_ld32(T_S(bb) + lane_addr + half * 32, sv);
      tmem_ld32(T_DP(bb) + lane_addr + half * 32, dv);
      tmem_ld_wait();
      uint32_t pp[16], dd[16];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 l4 = st_l[j], d4 = st_d[j];
        const float la[4] = {l4.x, l4.y, l4.z, l4.w}, da[4] = {d4.x, d4.y, d4.z, d4.w};
        float pv[4], dsv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float pr = fast_exp2(__uint_as_float(sv[4 * j + e]) * p.scale_log2 - la[e]);
          if (need_mask) {
            const int q = half * 32 + 4 * j + e;
            const bool vis = key_ok && q < qvalid && (!p.causal || kpos <= q0 + q);
            pr = vis ? pr : 0.f;
          }
          pv[e] = pr;
          dsv[e] = pr * (__uint_as_float(dv[4 * j + e]) - da[e]) * p.scale;
        }
        pp[2 * j] = pack_bf16(pv[0], pv[1]);
        pp[2 * j + 1] = pack_bf16(pv[2], pv[3]);
        dd[2 * j] = pack_bf16(dsv[0], dsv[1]);
        dd[2 * j + 1] = pack_bf16(dsv[2], dsv[3]);
      }
      // packed results go into the first 16 columns of this warp's own 32-column chunk
      tmem_st16(T_S(bb) + lane_addr + half * 32, pp);
      tmem_st16(T_DP(bb) + lane_addr + half * 32, dd);
      // dS^T row r, logical 16-byte chunks half*4 .. half*4+3, 128-byte swizzle
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int chunk = (half * 4 + j) ^ (r & 7);
        *reinterpret_cast<uint4*>(ds_row + chunk * 16) =
            make_uint4(dd[j * 4 + 0], dd[j * 4 + 1], dd[j * 4 + 2], dd[j * 4 + 3]);
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_ready[bb]);
    }
    if (ok) ok = mbar_wait(dkv_full, 0, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      // every lane runs the aligned TMEM loads; only the stores are predicated
      const long long grow = (long long)seq_start + (key_ok ? kpos : 0);
      bf16* dkp = p.dk + grow * p.dk_row_stride + (long long)g * HD + p.dh * kHD;
      bf16* dvp = p.dv + grow * p.dv_row_stride + (long long)g * HD + p.dh * kHD;
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        uint32_t a[32], bq[32];
        tmem_ld32(T_DK + lane_addr + c * 32, a);
        tmem_ld32(T_DV + lane_addr + c * 32, bq);
        tmem_ld_wait();
        if (key_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 x, y;
            x.x = pack_bf16(__uint_as_float(a[i * 8 + 0]), __uint_as_float(a[i * 8 + 1]));
            x.y = pack_bf16(__uint_as_float(a[i * 8 + 2]), __uint_as_float(a[i * 8 + 3]));
            x.z = pack_bf16(__uint_as_float(a[i * 8 + 4]), __uint_as_float(a[i * 8 + 5]));
            x.w = pack_bf16(__uint_as_float(a[i * 8 + 6]), __uint_as_float(a[i * 8 + 7]));
            y.x = pack_bf16(__uint_as_float(bq[i * 8 + 0]), __uint_as_float(bq[i * 8 + 1]));
            y.y = pack_bf16(__uint_as_float(bq[i * 8 + 2]), __uint_as_float(bq[i * 8 + 3]));
            y.z = pack_bf16(__uint_as_float(bq[i * 8 + 4]), __uint_as_float(bq[i * 8 + 5]));
            y.w = pack_bf16(__uint_as_float(bq[i * 8 + 6]), __uint_as_float(bq[i * 8 + 7]));
            *reinterpret_cast<uint4*>(dkp + c * 32 + i * 8) = x;
            *reinterpret_cast<uint4*>(dvp + c * 32 + i * 8) = y;
          }
        }
      }
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

// delta[h, row] = sum_d dO[row,h,d] * O[row,h,d]; one warp per (row, head).
__global__ void attn_bwd_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dout,
                                      float* __restrict__ delta, long long rows, int H, int HD,
                                      long long o_stride, long long do_stride) {
  const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= rows * H) return;
  const long long row = wid / H;
  const int h = (int)(wid - row * H);
  const bf16* op = o + row * o_stride + (long long)h * HD;
  const bf16* dp = dout + row * do_stride + (long long)h * HD;
  float s = 0.f;
  for (int i = lane * 2; i < HD; i += 64) {
    float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(op + i));
    float2 b2 = unpack_bf16(*reinterpret_cast<const uint32_t*>(dp + i));
    s += a.x * b2.x + a.y * b2.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[(long long)h * rows + row] = s;
}

}  // namespace ob

using namespace ob;

extern "C" {

// Gradients of packed-row attention (head_dim 128).
//   q, out, dout: [rows, H, 128];  k, v: [rows, G, 128]  (row strides in elements)
//   lse: [H, rows] from the forward;  delta: scratch [H, rows] fp32
//   dq_acc: scratch [rows, H, 128] fp32 (this call zeroes it);  dq: [rows, H, 128] bf16 out
//   dk, dv: [rows, G, 128] bf16 out with their own row strides
int ob_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                const int* cu_seqlens, int B, int max_seqlen, long long total_rows, int H, int G,
                int HD, long long q_row_stride, long long k_row_stride, long long v_row_stride,
                long long o_row_stride, long long do_row_stride, long long dk_row_stride,
                long long dv_row_stride, float scale, int causal, int* status,
                cudaStream_t stream) {
  if (B <= 0 || total_rows <= 0) return 0;
  if (HD != 128 && HD != 256) return 6005;
  if ((q_row_stride | k_row_stride | v_row_stride | do_row_stride | dk_row_stride | dv_row_stride) & 7)
    return 6001;
  {
    long long warps = total_rows * H;
    int threads = 256;
    long long blocks = (warps * 32 + threads - 1) / threads;
    attn_bwd_delta_kernel<<<(unsigned)blocks, threads, 0, stream>>>(
        (const bf16*)out, (const bf16*)dout, delta, total_rows, H, HD, o_row_stride, do_row_stride);
    OB_CHECK_LAUNCH();
  }
  cudaError_t me = cudaMemsetAsync(dq_acc, 0, (size_t)total_rows * H * HD * sizeof(float), stream);
  if (me != cudaSuccess) return 4100 + (int)me;
  CUtensorMap tmQ, tmK, tmV, tmDO, tmDQ;
  int e = make_tmap_3d(&tmQ, q, HD, H, total_rows, (uint64_t)HD * 2, (uint64_t)q_row_stride * 2, 64, 1, kQT);
  if (e) return 2000 + e;
  e = make_tmap_3d(&tmDO, dout, HD, H, total_rows, (uint64_t)HD * 2, (uint64_t)do_row_stride * 2, 64, 1, kQT);
  if (e) return 2500 + e;
  e = make_tmap_3d(&tmK, k, HD, G, total_rows, (uint64_t)HD * 2, (uint64_t)k_row_stride * 2, 64, 1, 128);
  if (e) return 3000 + e;
  e = make_tmap_3d(&tmV, v, HD, G, total_rows, (uint64_t)HD * 2, (uint64_t)v_row_stride * 2, 64, 1, 128);
  if (e) return 3500 + e;
  tmDQ = tmQ;   // only the 128-wide kernel adds dQ through a tensor map
  if (HD == 128) {
    e = make_tmap_2d(&tmDQ, dq_acc, total_rows, (uint64_t)H * HD, (uint64_t)H * HD, kQT, kHD, 4, false);
    if (e) return 1900 + e;
  }
  AttnBwdArgs a = {};
  a.cu_seqlens = cu_seqlens;
  a.lse = lse; a.delta = delta; a.dq_acc = dq_acc;
  a.dk = (bf16*)dk; a.dv = (bf16*)dv;
  a.dk_row_stride = dk_row_stride; a.dv_row_stride = dv_row_stride;
  a.total_rows = total_rows; a.H = H; a.G = G; a.causal = causal;
  a.scale = scale; a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  dim3 grid((max_seqlen + 127) / 128, G, B);
  if (HD == 128) {
    OB_ENSURE_DYN_SMEM(attn_bwd_kernel<128>, AttnBwdSmem<128>::kTotal);
    attn_bwd_kernel<128><<<grid, kBwdThreads, AttnBwdSmem<128>::kTotal, stream>>>(tmQ, tmK, tmV, tmDO, tmDQ, a);
    OB_CHECK_LAUNCH();
  } else {
    OB_ENSURE_DYN_SMEM(attn_bwd_kernel<256>, AttnBwdSmem<256>::kTotal);
    for (int dh = 0; dh < 2; ++dh) {   // one pass per 128-wide half of the head dimension
      a.dh = dh;
      attn_bwd_kernel<256><<<grid, kBwdThreads, AttnBwdSmem<256>::kTotal, stream>>>(tmQ, tmK, tmV, tmDO, tmDQ, a);
      OB_CHECK_LAUNCH();
    }
  }
  // fp32 accumulation buffer -> bf16 dq
  extern int ob_cast_f32_bf16(const float*, void*, long long, cudaStream_t);
  return ob_cast_f32_bf16(dq_acc, dq, total_rows * H * HD, stream);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Allocation-free variant (see attention_noalloc.h).  The work buffers of ob_attn_bwd live in
// this fixed device array: [0, 16 MiB) the fp32 dQ accumulator, then 128 KiB for delta.
#include "attention_noalloc.h"

namespace {
constexpr size_t kNoAllocDqBytes = (size_t)OB_ATTN_NOALLOC_MAX_ROW_HEADS * 128 * sizeof(float);
constexpr size_t kNoAllocDeltaBytes = (size_t)OB_ATTN_NOALLOC_MAX_ROW_HEADS * sizeof(float);
static __device__ __align__(256) unsigned char g_attn_noalloc_scratch[kNoAllocDqBytes + kNoAllocDeltaBytes];

// In host code the array's name is only a handle for the runtime, not a device address; the
// address is resolved once per device (with that device current) and cached here.
unsigned char* noalloc_scratch_for_current_device(int* err) {
  static unsigned char* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *err = 6101;
    return nullptr;
  }
  if (!cached[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_attn_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      *err = 6101;
      return nullptr;
    }
    cached[dev] = (unsigned char*)p;
  }
  *err = 0;
  return cached[dev];
}
}  // namespace

extern "C" int ob_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                   const float* lse, void* dq, void* dk, void* dv, const int* cu_seqlens, int B,
                                   int max_seqlen, long long total_rows, int H, int G, int HD,
                                   long long q_row_stride, long long k_row_stride, long long v_row_stride,
                                   long long o_row_stride, long long do_row_stride, long long dk_row_stride,
                                   long long dv_row_stride, float scale, int causal, int* status,
                                   cudaStream_t stream) {
  if (B <= 0 || total_rows <= 0) return 0;
  if (HD != 128) return 6005;   // the built-in scratch is laid out for 128-wide heads
  if (total_rows * (long long)H > OB_ATTN_NOALLOC_MAX_ROW_HEADS) return 6100;  // beyond the built-in scratch
  int err = 0;
  unsigned char* base = noalloc_scratch_for_current_device(&err);
  if (!base) return err;
  float* dq_acc = reinterpret_cast<float*>(base);
  float* delta = reinterpret_cast<float*>(base + kNoAllocDqBytes);
  // ob_attn_bwd zeroes dq_acc itself (cudaMemsetAsync on `stream`) and overwrites delta fully.
  return ob_attn_bwd(q, k, v, out, dout, lse, delta, dq_acc, dq, dk, dv, cu_seqlens, B, max_seqlen, total_rows, H,
                     G, HD, q_row_stride, k_row_stride, v_row_stride, o_row_stride, do_row_stride, dk_row_stride,
                     dv_row_stride, scale, causal, status, stream);
}
