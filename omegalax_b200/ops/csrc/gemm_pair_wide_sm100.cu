// K1, wide CTA-pair variant: one 512 x 256 output tile per cluster of two CTAs.
//
//   C[M,N] (+)= op(A) * op(B)^T       fp32 accumulation in TMEM, operand layouts as in gemm_sm100.cu
//
// Each CTA owns 256 rows of the tile as two 128-row halves and stages, per 64-deep k-block, its
// 256 rows of A (32 KB) and its 128 of the tile's 256 B rows (16 KB).  Per k-step the issuing
// thread of the even CTA runs two cta_group::2 MMAs (M 256 = one 128-row half from each CTA,
// N 256): half 0 into TMEM columns [0,256), half 1 into [256,512).  A k-block therefore moves
// 48 KB into each SM for 2 x 256 x 256 x 64 MACs: three quarters of the L2 -> shared-memory
// bytes per FLOP of the 256 x 256 pair tile, which is what leaves the shared-memory port to the
// tensor core (the 256 x 256 kernel tops out near 85 % tensor-pipe activity with the port shared
// evenly between TMA writes and operand reads).  No load is multicast.
//
// The two accumulators fill all 512 TMEM columns, so they cannot be double-buffered across tiles.
// The epilogue instead frees them quickly: warps 2..5 move each accumulator through a small
// 128-byte-swizzled staging ring in shared memory and hand it to the TMA unit (bulk tensor store,
// or bulk tensor reduce-add for the fp32-accumulate mode), releasing half 0 before half 1 so the
// next tile's first MMAs start while half 1 still drains.  Peer-reduction modes and outputs the
// TMA unit cannot address (pitch or base not 16-byte aligned) take the register -> global path.
//
// Roles per CTA (192 threads): warp 0 = TMA producer (both CTAs), warp 1 = TMEM allocation (both)
// and MMA issue (even CTA only), warps 2..5 = epilogue (both).  Barriers the issuing thread waits
// on live in the even CTA and are signalled across the pair.  Every wait is bounded.
#include "gemm_common.cuh"
#include "host_utils.h"

namespace ob {

constexpr int kWideStages = 4;
constexpr int kWideBM = 256;        // rows per CTA (two halves of 128)
constexpr int kWideBN = 256;        // tile columns
constexpr int kWideBNL = 128;       // B rows staged per CTA

struct WideSmem {
  static constexpr int kAHalf = 128 * BK * 2;            // 16 KB
  static constexpr int kABytes = 2 * kAHalf;
  static constexpr int kBBytes = kWideBNL * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;  // 48 KB
  static constexpr int kStagingOff = kWideStages * kStageBytes;   // 192 KB
  static constexpr int kStagingBytes = 4 * 2 * 4096;     // per epilogue warp: two 32-row x 128-byte slabs
  static constexpr int kBarOff = kStagingOff + kStagingBytes;
  static constexpr int kTotal = kBarOff + 256 + 1024;
};

struct WideTile {
  int row0;        // first of this CTA's 256 rows
  int b_row0;      // first B row (= output column) this CTA stages
  int c_col0;      // first output column of the tile
  int cols_valid;
};

__device__ __forceinline__ WideTile wide_tile(const GemmArgs& p, int t, int rank) {
  const int GM = p.raster_gm;
  const int per_group = GM * p.num_n_blocks;
  const int g = t / per_group;
  const int first_m = g * GM;
  const int gm = min(GM, p.num_m_blocks - first_m);
  const int r = t - g * per_group;
  const int mb = first_m + (r % gm);
  const int nb = r / gm;
  WideTile ti;
  ti.row0 = mb * 512 + rank * kWideBM;
  ti.b_row0 = nb * kWideBN + rank * kWideBNL;
  ti.c_col0 = nb * kWideBN;
  ti.cols_valid = min(kWideBN, p.N - ti.c_col0);
  return ti;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_bf16_pair_wide_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                           const __grid_constant__ CUtensorMap tmC, const GemmArgs p, const int tma_out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  using L = WideSmem;
  uint64_t* full_bar = (uint64_t*)(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + kWideStages;
  uint64_t* tfull_bar = empty_bar + kWideStages;     // [1]
  uint64_t* tempty_bar = tfull_bar + 1;              // [2], one per accumulator half
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank();
  const bool leader = rank == 0;
  const int pair0 = (int)(blockIdx.x >> 1);
  const int pair_step = (int)(gridDim.x >> 1);
  const int total_units = p.total_tiles * p.k_splits;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kWideStages; ++i) {
      mbar_init(&full_bar[i], 1);    // the even CTA's expect_tx arrival (bytes of both CTAs)
      mbar_init(&empty_bar[i], 1);   // one tcgen05.commit per CTA
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tempty_bar[0], 8);    // 4 epilogue warps of each CTA (used in the even CTA only)
    mbar_init(&tempty_bar[1], 8);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = pair0; u < total_units && ok; u += pair_step) {
        const int ks = u / p.total_tiles;        // slice-major: a wave of units shares operand panels
        const int t = u - ks * p.total_tiles;
        const int k_begin = ks * p.k_per_split;
        const int k_end = min(p.K, k_begin + p.k_per_split);
        const WideTile ti = wide_tile(p, t, rank);
        for (int k0 = k_begin; k0 < k_end; k0 += BK) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_EMPTY);
          if (!ok) break;
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * L::kStageBytes);
          const uint32_t fb = mapa_shared(smem_u32(&full_bar[stage]), 0);   // the even CTA's barrier
          if (!A_MN) {
            tma_load_2d_pair(sa, &tmA, fb, k0, ti.row0);                    // 256 rows x 64: both halves
          } else {
#pragma unroll
            for (int j = 0; j < kWideBM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tmA, fb, ti.row0 + j * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tmB, fb, k0, ti.b_row0);
          } else {
#pragma unroll
            for (int j = 0; j < kWideBNL / 64; ++j)
              tma_load_2d_pair(sb + j * (BK * 128), &tmB, fb, ti.b_row0 + j * 64, k0);
          }
          if (++stage == kWideStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_bf16(256, kWideBN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t tile_phase = 0;
      bool ok = true;
      for (int u = pair0; u < total_units && ok; u += pair_step) {
        const int ks = u / p.total_tiles;
        const int k_begin = ks * p.k_per_split;
        const int k_end = min(p.K, k_begin + p.k_per_split);
        uint32_t accumulate = 0;
        for (int k0 = k_begin; k0 < k_end && ok; k0 += BK) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, OB_ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (k0 == k_begin) {   // the previous tile's epilogue has drained this half
              ok = mbar_wait(&tempty_bar[h], tile_phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY);
              if (!ok) break;
              tc_fence_after();
            }
            const uint32_t sah = sa + h * L::kAHalf;
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              uint64_t adesc = A_MN ? make_smem_desc(sah + k * 2048, BK * 128, 1024) : make_smem_desc(sah + k * 32, 16, 1024);
              uint64_t bdesc = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
              umma_ss_pair(tmem_base + h * kWideBN, adesc, bdesc, idesc, (accumulate | (uint32_t)k) ? 1u : 0u);
            }
          }
          if (!ok) break;
          accumulate = 1;
          // the stage is free in both CTAs once these MMAs retire
          umma_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 0));
          umma_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 1));
          if (++stage == kWideStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (k_end <= k_begin) {   // nothing to accumulate: still hand the (unused) halves over in order
          for (int h = 0; h < 2 && ok; ++h)
            ok = mbar_wait(&tempty_bar[h], tile_phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY);
          if (!ok) break;
        }
        umma_commit_pair(mapa_shared(smem_u32(&tfull_bar[0]), 0));
        umma_commit_pair(mapa_shared(smem_u32(&tfull_bar[0]), 1));
        tile_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    uint8_t* stg = smem + L::kStagingOff + quad * 2 * 4096;
    const uint32_t my_row = smem_u32(stg) + lane * 128;
    const uint32_t sw = (uint32_t)(lane & 7);
    int buf = 0;
    uint32_t tile_phase = 0;
    bool ok = true;
    for (int u = pair0; u < total_units && ok; u += pair_step) {
      const int ks = u / p.total_tiles;
      const int t = u - ks * p.total_tiles;
      const bool empty_k = min(p.K, ks * p.k_per_split + p.k_per_split) <= ks * p.k_per_split;
      const WideTile ti = wide_tile(p, t, rank);
      ok = mbar_wait(&tfull_bar[0], tile_phase, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const int slab_row0 = ti.row0 + h * 128 + quad * 32;     // first row of this warp's 32-row slab
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + h * kWideBN;
        if (tma_out && p.out_mode == 0) {
          // bf16: 64 columns (128 bytes per row) per bulk tensor store
          const long long my_grow = (long long)slab_row0 + lane;
          const bool do_ce = p.ce_stats != nullptr && my_grow < p.M;
          const int tgt = do_ce ? __ldg(p.ce_targets + my_grow) : -1;
          float ce_m = -INFINITY, ce_s = 0.f;
#pragma unroll 1
          for (int cc = 0; cc < kWideBN / 64; ++cc) {
            uint32_t v0[32], v1[32];
            if (!empty_k) {
              tmem_ld32(taddr + cc * 64, v0);
              tmem_ld32(taddr + cc * 64 + 32, v1);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v0[i] = v1[i] = 0;
            }
            if (p.bias) {
              const int cb = ti.c_col0 + cc * 64;
              if (cb + 64 <= p.N) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  v0[i] = __float_as_uint(__uint_as_float(v0[i]) + __bfloat162float(__ldg(p.bias + cb + i)));
                  v1[i] = __float_as_uint(__uint_as_float(v1[i]) + __bfloat162float(__ldg(p.bias + cb + 32 + i)));
                }
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  if (cb + i < p.N) v0[i] = __float_as_uint(__uint_as_float(v0[i]) + __bfloat162float(__ldg(p.bias + cb + i)));
                  if (cb + 32 + i < p.N)
                    v1[i] = __float_as_uint(__uint_as_float(v1[i]) + __bfloat162float(__ldg(p.bias + cb + 32 + i)));
                }
              }
            }
            if (do_ce) {   // online maximum / sum of exponentials over this row's columns of the tile (fp32)
              const int cb = ti.c_col0 + cc * 64;
              const int nval = min(64, p.N - cb);
              if (nval > 0) {
                float mx = ce_m;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  if (i < nval) mx = fmaxf(mx, __uint_as_float(v0[i]));
                  if (32 + i < nval) mx = fmaxf(mx, __uint_as_float(v1[i]));
                }
                float acc = ce_s * fast_exp2((ce_m - mx) * 1.4426950408889634f);
                const float mb = mx * 1.4426950408889634f;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  if (i < nval) acc += fast_exp2(__uint_as_float(v0[i]) * 1.4426950408889634f - mb);
                  if (32 + i < nval) acc += fast_exp2(__uint_as_float(v1[i]) * 1.4426950408889634f - mb);
                }
                ce_m = mx;
                ce_s = acc;
                if (tgt >= cb && tgt < cb + 64) {
                  float tl = 0.f;
#pragma unroll
                  for (int i = 0; i < 32; ++i) {
                    if (cb + i == tgt) tl = __uint_as_float(v0[i]);
                    if (cb + 32 + i == tgt) tl = __uint_as_float(v1[i]);
                  }
                  p.ce_tgt[my_grow] = tl;
                }
              }
            }
            if (lane == 0) tma_store_wait_read<1>();   // the slab written two stores ago has been read
            __syncwarp();
            const uint32_t base = my_row + buf * 4096;
#pragma unroll
            for (int c = 0; c < 4; ++c)
              st_shared_v4(base + (((uint32_t)c ^ sw) << 4),
                           pack_bf16(__uint_as_float(v0[c * 8 + 0]), __uint_as_float(v0[c * 8 + 1])),
                           pack_bf16(__uint_as_float(v0[c * 8 + 2]), __uint_as_float(v0[c * 8 + 3])),
                           pack_bf16(__uint_as_float(v0[c * 8 + 4]), __uint_as_float(v0[c * 8 + 5])),
                           pack_bf16(__uint_as_float(v0[c * 8 + 6]), __uint_as_float(v0[c * 8 + 7])));
#pragma unroll
            for (int c = 0; c < 4; ++c)
              st_shared_v4(base + (((uint32_t)(c + 4) ^ sw) << 4),
                           pack_bf16(__uint_as_float(v1[c * 8 + 0]), __uint_as_float(v1[c * 8 + 1])),
                           pack_bf16(__uint_as_float(v1[c * 8 + 2]), __uint_as_float(v1[c * 8 + 3])),
                           pack_bf16(__uint_as_float(v1[c * 8 + 4]), __uint_as_float(v1[c * 8 + 5])),
                           pack_bf16(__uint_as_float(v1[c * 8 + 6]), __uint_as_float(v1[c * 8 + 7])));
            fence_proxy_async_smem();
            __syncwarp();
            const int col0 = ti.c_col0 + cc * 64;
            if (lane == 0) {   // a group is committed every time (empty when the slab lies outside C), so
                               // "at most one pending" above always means the other slab
              if (slab_row0 < p.M && col0 < p.N) tma_store_2d(&tmC, stg + buf * 4096, col0, slab_row0);
              tma_store_commit();
            }
            buf ^= 1;
          }
          if (do_ce) p.ce_stats[my_grow * p.num_n_blocks + (ti.c_col0 / kWideBN)] = make_float2(ce_m, ce_s);
        } else if (tma_out) {
          // fp32 store / accumulate: 32 columns (128 bytes per row) per bulk tensor store / reduce-add
#pragma unroll 1
          for (int c32 = 0; c32 < kWideBN / 32; ++c32) {
            uint32_t v[32];
            if (!empty_k) {
              tmem_ld32(taddr + c32 * 32, v);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = 0;
            }
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
            const uint32_t base = my_row + buf * 4096;
#pragma unroll
            for (int c = 0; c < 8; ++c)
              st_shared_v4(base + (((uint32_t)c ^ sw) << 4), v[c * 4 + 0], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            const int col0 = ti.c_col0 + c32 * 32;
            if (lane == 0) {
              if (slab_row0 < p.M && col0 < p.N && !(empty_k && p.out_mode == 2)) {
                if (p.out_mode == 2) tma_reduce_add_2d(&tmC, stg + buf * 4096, col0, slab_row0);
                else tma_store_2d(&tmC, stg + buf * 4096, col0, slab_row0);
              }
              tma_store_commit();
            }
            buf ^= 1;
          }
        } else {
          // register -> global path (peer reductions, residual, outputs the TMA unit cannot address)
          const long long grow = (long long)slab_row0 + lane;
          const bool row_ok = grow < p.M;
#pragma unroll 1
          for (int c = 0; c < kWideBN / 32; ++c) {
            uint32_t v[32];
            if (!empty_k) {
              tmem_ld32(taddr + c * 32, v);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = 0;
            }
            const int col0 = ti.c_col0 + c * 32;
            const int ncols = min(32, ti.cols_valid - c * 32);
            if (row_ok && ncols > 0) gemm_store_slice(p, 0, grow, col0, ncols, v);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[h]), 0));
      }
      tile_phase ^= 1;
    }
    if (lane == 0) tma_store_wait_all<0>();   // staged slabs have reached memory before shared memory goes away
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    long long t0 = clock64();
    while (clock64() - t0 < 2000000) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();   // nobody leaves while its partner may still signal its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <bool A_MN, bool B_MN>
static int launch_wide(const void* A, const void* B, GemmArgs args, long long a_rows, long long a_cols, long long lda,
                       long long b_rows, long long b_cols, long long ldb, int gm, int forced_splits,
                       cudaStream_t stream) {
  CUtensorMap tmA, tmB, tmC;
  int e;
  if (!A_MN) e = make_tmap_2d(&tmA, A, a_rows, a_cols, lda, kWideBM, BK);
  else e = make_tmap_2d(&tmA, A, a_rows, a_cols, lda, BK, 64);
  if (e) return 2000 + e;
  if (!B_MN) e = make_tmap_2d(&tmB, B, b_rows, b_cols, ldb, kWideBNL, BK);
  else e = make_tmap_2d(&tmB, B, b_rows, b_cols, ldb, BK, 64);
  if (e) return 3000 + e;
  // Output through the TMA unit when it can address it: local memory, no residual, 16-byte aligned
  // base and row pitch.
  int tma_out = 0;
  tmC = tmA;
  if (args.out_mode <= 2 && args.residual == nullptr && args.C != nullptr) {
    const int esz = args.out_mode == 0 ? 2 : 4;
    if (((uintptr_t)args.C & 15) == 0 && ((args.ldc * esz) & 15) == 0) {
      e = make_tmap_2d(&tmC, args.C, (uint64_t)args.M, (uint64_t)args.N, (uint64_t)args.ldc, 32, esz == 2 ? 64 : 32, esz);
      if (e == 0) tma_out = 1;
    }
  }
  auto kern = gemm_bf16_pair_wide_kernel<A_MN, B_MN>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_set[dev]) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WideSmem::kTotal);
    if (ce != cudaSuccess) return 4000 + (int)ce;
    attr_set[dev] = true;
  }
  static int max_pairs = 0;   // clusters of two that can be resident at once (one CTA per SM)
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_sms(), 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = WideSmem::kTotal;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) n = num_sms() / 2;
    (void)cudaGetLastError();
    max_pairs = n;
  }
  int pairs = max_pairs;
  args.raster_gm = gm;
  // reduction slices (reducing output modes only): fewest that fill the last wave to 95 %
  args.k_splits = 1;
  args.k_per_split = args.K > 0 ? ((args.K + BK - 1) / BK) * BK : BK;
  if (args.out_mode >= 2 && args.out_mode <= 4 && args.K >= 2048 && forced_splits != 0) {
    const int kblocks = (args.K + BK - 1) / BK;
    int best = 1;
    double best_eff = 0.0;
    for (int s = 1; s <= 16; ++s) {
      if (forced_splits > 0 && s != forced_splits) continue;
      const int per = (kblocks + s - 1) / s;
      if (s > 1 && per * BK < 1024) break;
      const int s_eff = (kblocks + per - 1) / per;
      const long long units = (long long)args.total_tiles * s_eff;
      const double eff = (double)units / (double)(((units + pairs - 1) / pairs) * pairs);
      if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
      if (best_eff >= 0.95 && forced_splits <= 0) break;
    }
    const int per = (kblocks + best - 1) / best;
    args.k_per_split = per * BK;
    args.k_splits = (kblocks + per - 1) / per;
  }
  if (pairs > args.total_tiles * args.k_splits) pairs = args.total_tiles * args.k_splits;
  if (pairs <= 0) return 0;
  if (args.ce_stats != nullptr && !(tma_out && args.out_mode == 0)) return 6008;   // statistics live in the TMA bf16 epilogue
  kern<<<2 * pairs, kGemmThreads, WideSmem::kTotal, stream>>>(tmA, tmB, tmC, args, tma_out);
  OB_CHECK_LAUNCH();
  return 0;
}

// Entry used by the pair launchers in gemm_pair_sm100.cu: `g` describes the GEMM (M, N, K, output
// mode, C / peer pointers); tile counts are recomputed for the 512 x 256 tile.
int launch_pair_wide(const void* A, const void* B, const GemmArgs& g_in, long long lda, long long ldb, int a_mn,
                     int b_mn, int gm, int forced_splits, cudaStream_t stream) {
  GemmArgs g = g_in;
  g.num_m_blocks = (g.M + 511) / 512;
  g.num_n_blocks = (g.N + kWideBN - 1) / kWideBN;
  g.total_tiles = g.num_m_blocks * g.num_n_blocks;
  const long long a_rows = a_mn ? g.K : g.M, a_cols = a_mn ? g.M : g.K;
  const long long b_rows = b_mn ? g.K : g.N, b_cols = b_mn ? g.N : g.K;
  if (!a_mn && !b_mn) return launch_wide<false, false>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, gm, forced_splits, stream);
  if (!a_mn && b_mn) return launch_wide<false, true>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, gm, forced_splits, stream);
  if (a_mn && b_mn) return launch_wide<true, true>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, gm, forced_splits, stream);
  return launch_wide<true, false>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, gm, forced_splits, stream);
}

}  // namespace ob
