// K1, CTA-pair variant: one 256 x 256 output tile per cluster of two CTAs (tcgen05 cta_group::2).
//
//   C[M,N] (+)= op(A) * op(B)^T       fp32 accumulation in TMEM, same operand layouts as gemm_sm100.cu
//
// Each CTA stages its own 128 rows of the A tile and its own 128 rows of the B tile (the MMA reads
// both CTAs' shared memory), so a k-block moves 32 KB into each SM for 2 x 128 x 256 x 64 MACs:
// two thirds of the shared-memory / L2 traffic per FLOP of the single-CTA 128 x 256 tile, and a
// six-stage ring fits.  No load is multicast: every CTA fetches what it needs itself.
//
// Roles per CTA (192 threads): warp 0 = TMA producer (both CTAs), warp 1 = TMEM allocation (both)
// and MMA issue (even CTA only), warps 2..5 = epilogue (both; each CTA drains its 128 rows).
// Barriers: the "stage full" and "accumulator empty" barriers that the issuing thread waits on
// live in the even CTA; the odd CTA's TMA loads and epilogue warps signal them through their
// shared::cluster addresses.  "Stage empty" and "accumulator full" are signalled in both CTAs by
// two tcgen05.commit, one per CTA.  Every wait is bounded.
#include "gemm_common.cuh"
#include "host_utils.h"

namespace ob {

constexpr int kPairStages = 6;
constexpr int kPairBN = 256;        // tile columns (per pair)
constexpr int kPairBNL = 128;       // B rows staged per CTA

struct PairSmem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = kPairBNL * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingOff = kPairStages * kStageBytes;   // 4 epilogue warps x 4 KB (coalesced peer output)
  static constexpr int kBarOff = kStagingOff + 4 * 4096;
  static constexpr int kTotal = kBarOff + 256 + 1024;
};

struct PairTile {
  int row0;        // first row of this CTA's half of the tile (A rows and C rows)
  int b_row0;      // first B row (= output column) this CTA stages
  int c_col0;      // first output column of the tile
  int rows_valid, cols_valid;
  int b_k_off;     // grouped rows with an MN-major B: row offset of the group's matrix
  int k_begin, k_end;   // grouped reduction: the group's rows
  long long c_off; // grouped reduction: element offset of the group's output
  bool valid;
};

__device__ __forceinline__ int pair_find_group(const int* offs, int G, int row) {
  int lo = 0, hi = G;  // invariant: offs[lo] <= row < offs[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(offs + mid) <= row) lo = mid; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ PairTile pair_tile(const GemmArgs& p, int t, int rank) {
  if (p.mode == 1) {
    // rows of A and C are ragged per group; every group boundary is a multiple of 256, so a pair
    // tile lies inside one group and reads that group's matrix of B
    PairTile ti;
    const int mb = t / p.num_n_blocks, nb = t - mb * p.num_n_blocks;
    const int row0 = mb * 256;
    ti.valid = row0 < __ldg(p.group_offsets + p.num_groups);
    const int g = ti.valid ? pair_find_group(p.group_offsets, p.num_groups, row0) : 0;
    ti.row0 = row0 + rank * 128;
    ti.rows_valid = 128;
    if (p.b_mn) { ti.b_row0 = nb * kPairBN + rank * kPairBNL; ti.b_k_off = g * p.b_group_rows; }
    else { ti.b_row0 = g * p.b_group_rows + nb * kPairBN + rank * kPairBNL; ti.b_k_off = 0; }
    ti.c_col0 = nb * kPairBN;
    ti.cols_valid = min(kPairBN, p.N - ti.c_col0);
    ti.k_begin = 0; ti.k_end = p.K; ti.c_off = 0;
    return ti;
  }
  if (p.mode == 2) {
    // per-group weight gradient: the reduction runs over the group's rows
    PairTile ti;
    const int per_group = p.num_m_blocks * p.num_n_blocks;
    const int g = t / per_group, r = t - g * per_group;
    const int mb = r / p.num_n_blocks, nb = r - mb * p.num_n_blocks;
    ti.valid = true;
    ti.row0 = mb * 256 + rank * 128;
    ti.b_row0 = nb * kPairBN + rank * kPairBNL;
    ti.b_k_off = 0;
    ti.c_col0 = nb * kPairBN;
    ti.rows_valid = min(128, p.M - ti.row0);
    ti.cols_valid = min(kPairBN, p.N - ti.c_col0);
    ti.k_begin = __ldg(p.group_offsets + g);
    ti.k_end = __ldg(p.group_offsets + g + 1);
    ti.c_off = (long long)g * p.c_group_stride;
    return ti;
  }
  // GM tile rows (GM * 256 output rows) share a sweep over the tile columns for L2 reuse
  const int GM = p.raster_gm;
  const int per_group = GM * p.num_n_blocks;
  const int g = t / per_group;
  const int first_m = g * GM;
  const int gm = min(GM, p.num_m_blocks - first_m);
  const int r = t - g * per_group;
  int mb = first_m + (r % gm);
  int nb = r / gm;
  if (p.ag_side == 2) {  // B is gathered: sweep the tile rows for 4 tile columns of one chunk at a time
    const int pg = GM * p.num_m_blocks;
    const int g2 = t / pg;
    const int first_n = g2 * GM;
    const int gn = min(GM, p.num_n_blocks - first_n);
    const int r2 = t - g2 * pg;
    nb = first_n + (r2 % gn);
    mb = r2 / gn;
    nb += p.ag_rank * (p.ag_rows_per_rank / kPairBN);
    if (nb >= p.num_n_blocks) nb -= p.num_n_blocks;
  } else if (p.ag_side == 1) {  // own chunk of A first, then the chunks in arrival order
    mb += p.ag_rank * (p.ag_rows_per_rank / 256);
    if (mb >= p.num_m_blocks) mb -= p.num_m_blocks;
  } else if (p.m_rot) {
    mb += p.m_rot;
    if (mb >= p.num_m_blocks) mb -= p.num_m_blocks;
  }
  PairTile ti;
  ti.row0 = mb * 256 + rank * 128;
  ti.b_row0 = nb * kPairBN + rank * kPairBNL;
  ti.c_col0 = nb * kPairBN;
  ti.rows_valid = min(128, p.M - ti.row0);
  ti.cols_valid = min(kPairBN, p.N - ti.c_col0);
  ti.b_k_off = 0; ti.k_begin = 0; ti.k_end = p.K; ti.c_off = 0; ti.valid = true;
  return ti;
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmL, const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  using L = PairSmem;
  uint64_t* full_bar = (uint64_t*)(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + kPairStages;
  uint64_t* tfull_bar = empty_bar + kPairStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank();
  const bool leader = rank == 0;
  // gather mode: the first clusters of the grid only move data (an even number of CTAs, so a
  // cluster is either all copy or all compute)
  const int ncopy = p.ag_side ? p.ag_copy_ctas : 0;
  if ((int)blockIdx.x < ncopy) {
    if (threadIdx.x == 0) ag_copy_role<(L::kStagingOff / 32768 < 6 ? L::kStagingOff / 32768 : 6)>(p, smem, full_bar, abort_flag);
    return;
  }
  const int pair0 = (int)((blockIdx.x - ncopy) >> 1);
  const int pair_step = (int)((gridDim.x - ncopy) >> 1);
  const int total_units = p.total_tiles * p.k_splits;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kPairStages; ++i) {
      mbar_init(&full_bar[i], 1);    // the even CTA's expect_tx arrival (bytes of both CTAs)
      mbar_init(&empty_bar[i], 1);   // one tcgen05.commit per CTA
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 8);  // 4 epilogue warps of each CTA (used in the even CTA only)
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 2 * kPairBN);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();   // both CTAs' barriers are initialised before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      if (p.ag_side) tma_prefetch_desc(&tmL);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t ag_seen = 0;
      bool ok = true;
      for (int u = pair0; u < total_units && ok; u += pair_step) {
        const int ks = u / p.total_tiles;        // slice-major: a wave of units shares operand panels
        const int t = u - ks * p.total_tiles;
        const PairTile ti = pair_tile(p, t, rank);
        if (!ti.valid) continue;
        const int k_begin = p.mode ? ti.k_begin : ks * p.k_per_split;
        const int k_end = p.mode ? ti.k_end : min(p.K, k_begin + p.k_per_split);
        bool ag_local = false;   // tile of this GPU's own chunk: read it where it already is
        int ag_row = 0;
        if (p.ag_side) {  // the chunk this CTA's part of the tile reads must have arrived
          const int row0 = p.ag_side == 1 ? ti.row0 : ti.b_row0;
          const int ch = row0 / p.ag_rows_per_rank;
          ag_local = ch == p.ag_rank;
          ag_row = row0 - ch * p.ag_rows_per_rank;
          if (!ag_local && !((ag_seen >> ch) & 1u)) {
            ok = flag_wait_ge<false>(p.ag_flags + ch, p.ag_target, OB_WAIT_CYCLES, p.status, OB_ERR_WAIT_FLAG);
            if (!ok) {
              *abort_flag = 1;
              break;
            }
            fence_proxy_async_all();
            ag_seen |= 1u << ch;
          }
        }
        for (int k0 = k_begin; k0 < k_end; k0 += BK) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_EMPTY);
          if (!ok) break;
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * L::kStageBytes);
          const uint32_t fb = mapa_shared(smem_u32(&full_bar[stage]), 0);   // the even CTA's barrier
          if (!A_MN) {
            if (ag_local && p.ag_side == 1) tma_load_2d_pair(sa, &tmL, fb, k0, ag_row);
            else tma_load_2d_pair(sa, &tmA, fb, k0, ti.row0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tmA, fb, ti.row0 + j * 64, k0);
          }
          if (!B_MN) {
            if (ag_local && p.ag_side == 2) tma_load_2d_pair(sb, &tmL, fb, k0, ag_row);
            else tma_load_2d_pair(sb, &tmB, fb, k0, ti.b_row0);
          } else {
#pragma unroll
            for (int j = 0; j < kPairBNL / 64; ++j)
              tma_load_2d_pair(sb + j * (BK * 128), &tmB, fb, ti.b_row0 + j * 64, ti.b_k_off + k0);
          }
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_bf16(256, kPairBN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int u = pair0; u < total_units && ok; u += pair_step) {
        const int ks = u / p.total_tiles;
        int k_begin = ks * p.k_per_split;
        int k_end = min(p.K, k_begin + p.k_per_split);
        if (p.mode) {
          const PairTile ti = pair_tile(p, u - ks * p.total_tiles, 0);
          if (!ti.valid) continue;
          k_begin = ti.k_begin; k_end = ti.k_end;
        }
        ok = mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kPairBN;
        uint32_t accumulate = 0;
        for (int k0 = k_begin; k0 < k_end; k0 += BK) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, OB_ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            uint64_t adesc = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            uint64_t bdesc = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            umma_ss_pair(d_tmem, adesc, bdesc, idesc, accumulate);
            accumulate = 1;
          }
          // the stage is free in both CTAs once these MMAs retire
          umma_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 0));
          umma_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 1));
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(mapa_shared(smem_u32(&tfull_bar[acc]), 0));
        umma_commit_pair(mapa_shared(smem_u32(&tfull_bar[acc]), 1));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    // peer output modes with 16-byte aligned row segments go through the coalescing slab
    const bool peer_coalesced = p.out_mode >= 3 && p.mode == 0 &&
                                ((p.ldc * (p.out_mode == 3 ? 4 : 2)) & 15) == 0 &&
                                ((reinterpret_cast<uintptr_t>(p.peer_ptr[0]) & 15) == 0);
    for (int u = pair0; u < total_units && ok; u += pair_step) {
      const int t = u % p.total_tiles;
      const PairTile ti = pair_tile(p, t, rank);
      if (!ti.valid) continue;
      const bool empty_k = p.mode ? (ti.k_end <= ti.k_begin) : (p.K <= 0);
      ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const int r = quad * 32 + lane;
      const bool row_ok = r < ti.rows_valid;
      const long long grow = (long long)ti.row0 + r;
#pragma unroll 1
      for (int c = 0; c < kPairBN / 32; ++c) {
        uint32_t v[32];
        if (!empty_k) {
          tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + acc * kPairBN + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        const int col0 = ti.c_col0 + c * 32;
        const int ncols = min(32, ti.cols_valid - c * 32);
        if (peer_coalesced && ncols == 32) {   // warp-uniform: rows owned by other GPUs leave as whole row segments
          peer_chunk_out(p, smem + L::kStagingOff + quad * 4096, lane, (long long)ti.row0 + quad * 32, col0, v);
        } else if (row_ok && ncols > 0) {
          gemm_store_slice(p, ti.c_off, grow, col0, ncols, v);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[acc]), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
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
    tmem_dealloc_pair(tmem_base, 2 * kPairBN);
  }
}

// Process-wide tuning knobs (ob_gemm_pair_tune): -1 = decide per launch.
static int g_tune_gm = -1, g_tune_wide = -1, g_tune_splitk = -1;

// gemm_pair_wide_sm100.cu
int launch_pair_wide(const void* A, const void* B, const GemmArgs& g, long long lda, long long ldb, int a_mn, int b_mn,
                     int gm, int forced_splits, cudaStream_t stream);

// The 512 x 256 tile kernel serves plain GEMMs into this GPU's memory without a fused residual whose
// tile count fills the SM pairs at least twice over (or whose reduction can be split to that
// effect).  Outputs that travel over NVLink from the epilogue (peer reductions / peer stores) stay on
// the 256 x 256 kernel: a CTA's fair share of the link is a few GB/s, so draining a tile takes tens
// of microseconds, which the double-buffered accumulators of that kernel hide behind the next tile's
// main loop and the single accumulator set of the wide kernel would not.
static bool want_wide(const GemmArgs& g) {
  if (g_tune_wide == 0) return false;
  if (g.residual != nullptr || g.ag_side != 0 || g.mode != 0) return false;
  if (g.bias != nullptr && g.out_mode != 0) return false;   // its fp32 TMA epilogue adds no bias
  if (g_tune_wide == 1) return true;
  if (g.out_mode >= 3) return false;
  const long long tiles = (long long)((g.M + 511) / 512) * ((g.N + 255) / 256);
  if (g.out_mode >= 2 && g.out_mode <= 4) return tiles * (g.K / 1024 > 0 ? g.K / 1024 : 1) >= 148;
  return tiles >= 296;
}

// Tile rows per raster group: as many as keep the group's A panels (GM x 256 rows x K) within
// about 24 MB of L2 while the B panels stream past, between 2 and 16.
static int pick_gm(int K) {
  if (g_tune_gm > 0) return g_tune_gm;
  const long long panel = 256ll * (K > 0 ? K : 1) * 2;
  int gm = 2;
  while (gm < 16 && (long long)(2 * gm) * panel <= (24ll << 20)) gm *= 2;
  return gm;
}

// Slices of the reduction for the reducing output modes: the fewest that fill the last wave of
// the `pairs` resident clusters to 95 % (every slice at least 1024 deep), at most 8.
static void pick_splits(GemmArgs& g, int pairs) {
  g.k_splits = 1;
  g.k_per_split = g.K > 0 ? g.K : BK;
  if (g.mode != 0 || g.out_mode < 2 || g.out_mode > 4 || g.K < 2048 || g_tune_splitk == 0 || pairs <= 0) return;
  const int kblocks = (g.K + BK - 1) / BK;
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= 8; ++s) {
    if (g_tune_splitk > 0 && s != g_tune_splitk) continue;
    const int per = (kblocks + s - 1) / s;
    if (s > 1 && per * BK < 1024) break;
    const int s_eff = (kblocks + per - 1) / per;
    const long long units = (long long)g.total_tiles * s_eff;
    const double eff = (double)units / (double)(((units + pairs - 1) / pairs) * pairs);
    if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
    if (best_eff >= 0.95 && g_tune_splitk <= 0) break;
  }
  const int per = (kblocks + best - 1) / best;
  g.k_per_split = per * BK;
  g.k_splits = (kblocks + per - 1) / per;
}

template <bool A_MN, bool B_MN>
static int launch_pair(const void* A, const void* B, const GemmArgs& args_in, long long a_rows, long long a_cols,
                       long long lda, long long b_rows, long long b_cols, long long ldb, cudaStream_t stream) {
  GemmArgs args = args_in;
  CUtensorMap tmA, tmB;
  int e;
  if (!A_MN) e = make_tmap_2d(&tmA, A, a_rows, a_cols, lda, BM, BK);
  else e = make_tmap_2d(&tmA, A, a_rows, a_cols, lda, BK, 64);
  if (e) return 2000 + e;
  if (!B_MN) e = make_tmap_2d(&tmB, B, b_rows, b_cols, ldb, kPairBNL, BK);
  else e = make_tmap_2d(&tmB, B, b_rows, b_cols, ldb, BK, 64);
  if (e) return 3000 + e;
  CUtensorMap tmL = tmA;  // gather mode: this GPU's own chunk of the gathered operand, in place
  if (args.ag_side) {
    e = make_tmap_2d(&tmL, args.ag_src[args.ag_rank], args.ag_rows_per_rank, args.K, args.K,
                     args.ag_side == 1 ? BM : kPairBNL, BK);
    if (e) return 3500 + e;
  }
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN>;
  OB_ENSURE_DYN_SMEM(kern, PairSmem::kTotal);
  static int max_pairs = 0;   // clusters of two that can be resident at once (one CTA per SM)
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_sms(), 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = PairSmem::kTotal;
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
  int copy = 0;
  if (args.ag_side) {  // copy clusters come first in the grid; every cluster is resident from the start
    copy = args.ag_copy_ctas;
    pairs -= copy / 2;
  }
  args.raster_gm = pick_gm(args.K);
  pick_splits(args, pairs);
  if (pairs > args.total_tiles * args.k_splits) pairs = args.total_tiles * args.k_splits;
  if (pairs <= 0) return args.ag_side ? 6006 : 0;
  kern<<<2 * pairs + copy, kGemmThreads, PairSmem::kTotal, stream>>>(tmA, tmB, tmL, args);
  OB_CHECK_LAUNCH();
  return 0;
}

}  // namespace ob

using namespace ob;

extern "C" {

// Tuning knobs of the CTA-pair kernel for the whole process; -1 restores the per-launch choice.
// gm: tile rows per raster group; wide: 0 never / 1 always use the 512 x 256 tile kernel where it
// applies; splitk: 0 never split the reduction, n > 0 always n slices (reducing output modes only).
void ob_gemm_pair_tune(int gm, int wide, int splitk) {
  g_tune_gm = gm; g_tune_wide = wide; g_tune_splitk = splitk;
}

// Same contract as ob_gemm_bf16 (plain mode), computed by CTA pairs on 256 x 256 tiles.
// bias (optional, bf16 [N]) is added before the store; ce_targets / ce_stats / ce_tgt (optional, bf16
// output only) request the cross-entropy statistics epilogue of the 512 x 256 tile kernel.
int ob_gemm_bf16_pair(const void* A, const void* B, void* C, const void* residual, int M, int N, int K, long long lda,
                      long long ldb, long long ldc, long long ldr, int a_mn, int b_mn, int out_mode, const void* bias,
                      const int* ce_targets, void* ce_stats, float* ce_tgt, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((lda & 7) || (ldb & 7)) return 6001;
  if ((((uintptr_t)A) & 15) || (((uintptr_t)B) & 15)) return 6002;
  if (out_mode < 0 || out_mode > 2) return 6005;
  GemmArgs g = {};
  g.M = M; g.N = N; g.K = K; g.mode = 0;
  g.num_m_blocks = (M + 255) / 256;
  g.num_n_blocks = (N + kPairBN - 1) / kPairBN;
  g.total_tiles = g.num_m_blocks * g.num_n_blocks;
  g.C = C; g.ldc = ldc; g.out_mode = out_mode;
  g.residual = (const bf16*)residual; g.ldr = ldr;
  g.bias = (const bf16*)bias;
  g.ce_targets = ce_targets; g.ce_stats = (float2*)ce_stats; g.ce_tgt = ce_tgt;
  g.status = status;
  if (ce_stats != nullptr) {
    if (out_mode != 0 || residual != nullptr) return 6008;
    return launch_pair_wide(A, B, g, lda, ldb, a_mn, b_mn, pick_gm(2 * K), 0, stream);
  }
  if (want_wide(g)) return launch_pair_wide(A, B, g, lda, ldb, a_mn, b_mn, pick_gm(2 * K), g_tune_splitk, stream);
  const long long a_rows = a_mn ? K : M, a_cols = a_mn ? M : K;
  const long long b_rows = b_mn ? K : N, b_cols = b_mn ? N : K;
  if (!a_mn && !b_mn) return launch_pair<false, false>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, stream);
  if (!a_mn && b_mn) return launch_pair<false, true>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, stream);
  if (a_mn && b_mn) return launch_pair<true, true>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, stream);
  return launch_pair<true, false>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, stream);
}

// Same contract as ob_gemm_bf16_peer_reduce (fp32 result rows added into the owning GPUs' buffers
// with vector reductions over NVLink), computed by CTA pairs.
// bf16_out: 0 fp32 reduction, 1 bf16 reduction, 2 + s = bf16 store into slab s of the owner's staging
// buffer (first phase of the two-phase reduce-scatter; the owner sums the slabs afterwards).
int ob_gemm_bf16_pair_peer_reduce(const void* A, const void* B, void* const* peer_ptrs, int world, int rows_per_peer,
                                  int M, int N, int K, long long lda, long long ldb, long long ldc, int a_mn, int b_mn,
                                  int bf16_out, int first_owner, int* status, cudaStream_t stream) {
  if (world > kMaxPeers) return 6003;
  if ((lda & 7) || (ldb & 7)) return 6001;
  GemmArgs g = {};
  g.M = M; g.N = N; g.K = K; g.mode = 0;
  g.num_m_blocks = (M + 255) / 256;
  if (first_owner > 0 && first_owner < world)
    g.m_rot = (int)(((long long)first_owner * rows_per_peer / 256) % g.num_m_blocks);
  g.num_n_blocks = (N + kPairBN - 1) / kPairBN;
  g.total_tiles = g.num_m_blocks * g.num_n_blocks;
  g.C = nullptr; g.ldc = ldc; g.out_mode = bf16_out >= 2 ? 5 : bf16_out ? 4 : 3;
  g.peer_slot = bf16_out >= 2 ? bf16_out - 2 : 0;
  for (int i = 0; i < world; ++i) g.peer_ptr[i] = (float*)peer_ptrs[i];
  g.rows_per_peer = rows_per_peer;
  g.status = status;
  if (want_wide(g)) return launch_pair_wide(A, B, g, lda, ldb, a_mn, b_mn, pick_gm(2 * K), g_tune_splitk, stream);
  const long long a_rows = a_mn ? K : M, a_cols = a_mn ? M : K;
  const long long b_rows = b_mn ? K : N, b_cols = b_mn ? N : K;
  if (!a_mn && !b_mn) return launch_pair<false, false>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, stream);
  if (!a_mn && b_mn) return launch_pair<false, true>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, stream);
  if (a_mn && b_mn) return launch_pair<true, true>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, stream);
  return launch_pair<true, false>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, stream);
}

// Grouped GEMM over ragged row groups on CTA pairs (mixture-of-experts forward and input gradient):
// same contract as ob_gemm_bf16_grouped, but every entry of group_offsets and max_rows must be a
// multiple of 256 (a 256-row pair tile must not straddle two groups).
int ob_gemm_bf16_pair_grouped(const void* A, const void* B, void* C, const int* group_offsets, int G, int max_rows,
                              int N, int K, long long lda, long long ldc, int b_mn, int out_mode, int* status,
                              cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if ((lda & 7) || (max_rows % 256)) return 6001;
  GemmArgs g = {};
  g.M = max_rows; g.N = N; g.K = K; g.mode = 1;
  g.num_groups = G; g.group_offsets = group_offsets;
  g.b_group_rows = b_mn ? K : N;
  g.b_mn = b_mn;
  g.num_m_blocks = max_rows / 256;
  g.num_n_blocks = (N + kPairBN - 1) / kPairBN;
  g.total_tiles = g.num_m_blocks * g.num_n_blocks;
  g.C = C; g.ldc = ldc; g.out_mode = out_mode;
  g.status = status;
  const long long b_rows = (long long)G * (b_mn ? K : N), b_cols = b_mn ? N : K;
  if (b_mn) return launch_pair<false, true>(A, B, g, max_rows, K, lda, b_rows, b_cols, b_cols, stream);
  return launch_pair<false, false>(A, B, g, max_rows, K, lda, b_rows, b_cols, b_cols, stream);
}

// Grouped weight gradient on CTA pairs: same contract as ob_gemm_bf16_grouped_wgrad.
int ob_gemm_bf16_pair_grouped_wgrad(const void* A, const void* B, void* C, const int* group_offsets, int G,
                                    int max_rows, int N, int K, long long lda, long long ldb, int out_mode, int* status,
                                    cudaStream_t stream) {
  if ((lda & 7) || (ldb & 7)) return 6001;
  GemmArgs g = {};
  g.M = N; g.N = K; g.K = max_rows; g.mode = 2;
  g.num_groups = G; g.group_offsets = group_offsets;
  g.num_m_blocks = (N + 255) / 256;
  g.num_n_blocks = (K + kPairBN - 1) / kPairBN;
  g.total_tiles = G * g.num_m_blocks * g.num_n_blocks;
  g.C = C; g.ldc = K; g.c_group_stride = (long long)N * K; g.out_mode = out_mode;
  g.status = status;
  return launch_pair<true, true>(A, B, g, max_rows, N, lda, max_rows, K, ldb, stream);
}

// Same contract as ob_gemm_bf16_ag (all-gather -> GEMM in one launch), computed by CTA pairs.  The
// chunk of each rank must be a multiple of 256 rows and copy_ctas even.
int ob_gemm_bf16_pair_ag(const void* other, void* full, void* const* src_ptrs, void* C, const void* residual, int M,
                         int N, int K, long long ldc, long long ldr, int out_mode, int side, int world, int rank,
                         int rows_per_rank, unsigned* flags, unsigned target, int copy_ctas, int* status,
                         cudaStream_t stream) {
  if (world > kMaxPeers || world <= 0 || copy_ctas <= 0 || copy_ctas > 32 || (copy_ctas & 1)) return 6003;
  if (side != 1 && side != 2) return 6005;
  if ((K & 7) || (rows_per_rank % 256)) return 6007;
  if ((long long)rows_per_rank * world != (side == 1 ? M : N)) return 6007;
  GemmArgs g = {};
  g.M = M; g.N = N; g.K = K; g.mode = 0;
  g.num_m_blocks = (M + 255) / 256;
  g.num_n_blocks = (N + kPairBN - 1) / kPairBN;
  g.total_tiles = g.num_m_blocks * g.num_n_blocks;
  g.C = C; g.ldc = ldc; g.out_mode = out_mode;
  g.residual = (const bf16*)residual; g.ldr = ldr;
  g.ag_side = side; g.ag_world = world; g.ag_rank = rank; g.ag_copy_ctas = copy_ctas;
  g.ag_rows_per_rank = rows_per_rank;
  for (int i = 0; i < world; ++i) g.ag_src[i] = src_ptrs[i];
  g.ag_dst = full;
  g.ag_chunk_bytes = (long long)rows_per_rank * K * 2;
  g.ag_flags = flags; g.ag_target = target;
  g.status = status;
  const void* A = side == 1 ? full : other;
  const void* B = side == 2 ? full : other;
  return launch_pair<false, false>(A, B, g, M, K, K, N, K, K, stream);
}

}  // extern "C"
