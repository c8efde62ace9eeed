// K1/K2: persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] (+)= op(A) * op(B)^T      fp32 accumulation in TMEM
//
// Roles inside one CTA (192 threads): warp 0 issues TMA loads into a 4-stage ring of
// 128-byte-swizzled shared-memory tiles, warp 1 allocates TMEM and issues tcgen05.mma
// (one thread), warps 2..5 drain the accumulator with tcgen05.ld and run the epilogue.
// Two accumulators of BN columns each are kept in TMEM so the epilogue of tile i
// overlaps the main loop of tile i+1.  One CTA per SM, persistent over output tiles.
//
// Operand storage ("major-ness"), per operand:
//   K-major : reduction dimension contiguous.  A is [M,K] row-major, B is [N,K] row-major.
//   MN-major: output dimension contiguous.     A is [K,M] row-major, B is [K,N] row-major.
// The three training GEMMs of a linear layer y = x W^T map to
//   fprop  y  = x  W^T : A=x  (K-major),  B=W  (K-major)
//   dgrad  dx = dy W   : A=dy (K-major),  B=W  (MN-major, reduction over W's rows)
//   wgrad  dW = dy^T x : A=dy (MN-major), B=x  (MN-major, reduction over tokens)
//
// Grouped modes (mixture-of-experts):
//   mode 1: rows of A and C are ragged per group (group_offsets, multiples of 128);
//           B holds one matrix per group, stacked along its row dimension.
//   mode 2: per-group weight gradient; the reduction runs over the group's rows.
//
// Output modes: bf16 store, fp32 store, fp32 accumulate (C += result), optional bf16
// residual added before the store, and a peer-reduce mode in which row blocks of C are
// owned by other GPUs and the tile is added there with vector red.global.add (used by the
// fused GEMM -> reduce-scatter paths over NVLink peer memory).
//
// Gather mode (all-gather -> GEMM in one launch): one K-major operand is spread over the GPUs in
// equal row chunks.  The first few CTAs of the grid do not compute: one thread of each streams
// its share of every chunk from the owner's memory (bulk copies, peer memory included) through a
// ring of shared-memory buffers into this GPU's full operand and bumps a per-chunk counter.  The
// TMA producer of a computing CTA waits (bounded) for the counter of the chunk its tile reads;
// tiles are visited own chunk first, then in the order the chunks arrive.
#include "gemm_common.cuh"
#include "host_utils.h"

namespace ob {

__device__ __forceinline__ int find_group(const int* offs, int G, int row) {
  int lo = 0, hi = G;  // invariant: offs[lo] <= row < offs[hi] (if row < offs[G])
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (__ldg(offs + mid) <= row) lo = mid; else hi = mid;
  }
  return lo;
}

template <int BN>
__device__ __forceinline__ TileInfo get_tile(const GemmArgs& p, int t) {
  TileInfo ti;
  ti.valid = true;
  ti.c_off = 0;
  ti.b_k_off = 0;
  if (p.mode == 0) {
    // grouped raster: 8 row blocks share a sweep over the column blocks for L2 reuse
    const int GM = 8;
    int mb, nb;
    if (p.ag_side != 2) {
      int per_group = GM * p.num_n_blocks;
      int g = t / per_group;
      int first_m = g * GM;
      int gm = min(GM, p.num_m_blocks - first_m);
      int r = t - g * per_group;
      mb = first_m + (r % gm);
      nb = r / gm;
      if (p.ag_side == 1) {  // own chunk of A first, then the chunks in arrival order
        mb += p.ag_rank * (p.ag_rows_per_rank / BM);
        if (mb >= p.num_m_blocks) mb -= p.num_m_blocks;
      } else if (p.m_rot) {
        mb += p.m_rot;
        if (mb >= p.num_m_blocks) mb -= p.num_m_blocks;
      }
    } else {  // B is gathered: sweep the row blocks for 8 column blocks of one chunk at a time
      int per_group = GM * p.num_m_blocks;
      int g = t / per_group;
      int first_n = g * GM;
      int gn = min(GM, p.num_n_blocks - first_n);
      int r = t - g * per_group;
      nb = first_n + (r % gn);
      mb = r / gn;
      nb += p.ag_rank * (p.ag_rows_per_rank / BN);
      if (nb >= p.num_n_blocks) nb -= p.num_n_blocks;
    }
    ti.a_row0 = mb * BM;
    ti.b_row0 = nb * BN;
    ti.c_row0 = mb * BM;
    ti.c_col0 = nb * BN;
    ti.rows_valid = min(BM, p.M - ti.c_row0);
    ti.cols_valid = min(BN, p.N - ti.c_col0);
    ti.k_begin = 0;
    ti.k_end = p.K;
  } else if (p.mode == 1) {
    int mb = t / p.num_n_blocks;
    int nb = t - mb * p.num_n_blocks;
    int row0 = mb * BM;
    int total = __ldg(p.group_offsets + p.num_groups);
    if (row0 >= total) {
      ti.valid = false;
      return ti;
    }
    int g = find_group(p.group_offsets, p.num_groups, row0);
    ti.a_row0 = row0;
    if (p.b_mn) {
      ti.b_row0 = nb * BN;
      ti.b_k_off = g * p.b_group_rows;
    } else {
      ti.b_row0 = g * p.b_group_rows + nb * BN;
    }
    ti.c_row0 = row0;
    ti.c_col0 = nb * BN;
    ti.rows_valid = BM;
    ti.cols_valid = min(BN, p.N - ti.c_col0);
    ti.k_begin = 0;
    ti.k_end = p.K;
  } else {
    int per_group = p.num_m_blocks * p.num_n_blocks;
    int g = t / per_group;
    int r = t - g * per_group;
    int mb = r / p.num_n_blocks;
    int nb = r - mb * p.num_n_blocks;
    ti.a_row0 = mb * BM;
    ti.b_row0 = nb * BN;
    ti.c_row0 = mb * BM;
    ti.c_col0 = nb * BN;
    ti.rows_valid = min(BM, p.M - ti.c_row0);
    ti.cols_valid = min(BN, p.N - ti.c_col0);
    ti.k_begin = __ldg(p.group_offsets + g);
    ti.k_end = __ldg(p.group_offsets + g + 1);
    ti.c_off = (long long)g * p.c_group_stride;
  }
  return ti;
}

template <int BN>
struct GemmSmem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOff = kStages * kStageBytes;
  static constexpr int kTotal = kBarOff + 256 + 1024;  // barriers + alignment slack
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmL, const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits.
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  using L = GemmSmem<BN>;
  uint64_t* full_bar = (uint64_t*)(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int ncopy = p.ag_side ? p.ag_copy_ctas : 0;
  if ((int)blockIdx.x < ncopy) {  // gather mode: this CTA only moves data
    // the copy ring lives in the stage area: 6 slots under a 192 KB ring, 4 under the 128 KB one
    if (threadIdx.x == 0) ag_copy_role<(L::kBarOff / 32768 < 6 ? L::kBarOff / 32768 : 6)>(p, smem, full_bar, abort_flag);
    return;
  }
  const int cta0 = (int)blockIdx.x - ncopy;
  const int cta_step = (int)gridDim.x - ncopy;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      if (p.ag_side) tma_prefetch_desc(&tmL);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t ag_seen = 0;
      bool ok = true;
      for (int t = cta0; t < p.total_tiles && ok; t += cta_step) {
        TileInfo ti = get_tile<BN>(p, t);
        if (!ti.valid) continue;
        bool ag_local = false;   // tile of this GPU's own chunk: read it where it already is
        int ag_row = 0;
        if (p.ag_side) {  // the chunk this tile reads must have arrived
          const int row0 = p.ag_side == 1 ? ti.a_row0 : ti.b_row0;
          const int ch = row0 / p.ag_rows_per_rank;
          ag_local = ch == p.ag_rank;
          ag_row = row0 - ch * p.ag_rows_per_rank;
          if (!ag_local && !((ag_seen >> ch) & 1u)) {
            ok = flag_wait_ge<false>(p.ag_flags + ch, p.ag_target, OB_WAIT_CYCLES, p.status, OB_ERR_WAIT_FLAG);
            if (!ok) {
              *abort_flag = 1;
              break;
            }
            fence_proxy_async_all();  // written through the generic / bulk path, read by TMA next
            ag_seen |= 1u << ch;
          }
        }
        for (int k0 = ti.k_begin; k0 < ti.k_end; k0 += BK) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_EMPTY);
          if (!ok) break;
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          if (!A_MN) {
            if (ag_local && p.ag_side == 1) tma_load_2d(sa, &tmL, &full_bar[stage], k0, ag_row);
            else tma_load_2d(sa, &tmA, &full_bar[stage], k0, ti.a_row0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), &tmA, &full_bar[stage], ti.a_row0 + j * 64, k0);
          }
          if (!B_MN) {
            if (ag_local && p.ag_side == 2) tma_load_2d(sb, &tmL, &full_bar[stage], k0, ag_row);
            else tma_load_2d(sb, &tmB, &full_bar[stage], k0, ti.b_row0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), &tmB, &full_bar[stage], ti.b_row0 + j * 64,
                          ti.b_k_off + k0);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = cta0; t < p.total_tiles && ok; t += cta_step) {
        TileInfo ti = get_tile<BN>(p, t);
        if (!ti.valid) continue;
        ok = mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status,
                       OB_ERR_WAIT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        uint32_t accumulate = 0;
        for (int k0 = ti.k_begin; k0 < ti.k_end; k0 += BK) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, OB_ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            uint64_t adesc = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024)
                                  : make_smem_desc(sa + k * 32, 16, 1024);
            uint64_t bdesc = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024)
                                  : make_smem_desc(sb + k * 32, 16, 1024);
            umma_ss(d_tmem, adesc, bdesc, idesc, accumulate);
            accumulate = 1;
          }
          umma_commit(&empty_bar[stage]);  // stage is free once these MMAs retire
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = cta0; t < p.total_tiles && ok; t += cta_step) {
      TileInfo ti = get_tile<BN>(p, t);
      if (!ti.valid) continue;
      ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const int r = quad * 32 + lane;
      const bool row_ok = r < ti.rows_valid;
      const long long grow = (long long)ti.c_row0 + r;
      const bool empty_k = ti.k_end <= ti.k_begin;  // nothing was accumulated: result is zero
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        if (!empty_k) {
          tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        const int col0 = ti.c_col0 + c * 32;
        const int ncols = min(32, ti.cols_valid - c * 32);
        if (row_ok && ncols > 0) gemm_store_slice(p, ti.c_off, grow, col0, ncols, v);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
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
    // give copies that may still be in flight time to land before shared memory is released
    long long t0 = clock64();
    while (clock64() - t0 < 2000000) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const void* A, const void* B, const GemmArgs& args, long long a_rows,
                       long long a_cols, long long lda, long long b_rows, long long b_cols,
                       long long ldb, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  // K-major operand: view [rows=MN extent, cols=K], box BM(BN) x 64.
  // MN-major operand: view [rows=K extent, cols=MN], box 64 (k) x 64 (mn).
  int e;
  if (!A_MN) e = make_tmap_2d(&tmA, A, a_rows, a_cols, lda, BM, BK);
  else e = make_tmap_2d(&tmA, A, a_rows, a_cols, lda, BK, 64);
  if (e) return 2000 + e;
  if (!B_MN) e = make_tmap_2d(&tmB, B, b_rows, b_cols, ldb, BN, BK);
  else e = make_tmap_2d(&tmB, B, b_rows, b_cols, ldb, BK, 64);
  if (e) return 3000 + e;
  CUtensorMap tmL = tmA;  // gather mode: this GPU's own chunk of the gathered operand, in place
  if (args.ag_side) {
    e = make_tmap_2d(&tmL, args.ag_src[args.ag_rank], args.ag_rows_per_rank, args.K, args.K,
                     args.ag_side == 1 ? BM : BN, BK);
    if (e) return 3500 + e;
  }
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  OB_ENSURE_DYN_SMEM(kern, GemmSmem<BN>::kTotal);
  int grid = args.total_tiles < num_sms() ? args.total_tiles : num_sms();
  if (grid <= 0) return 0;
  if (args.ag_side) {  // copy CTAs come first in the grid; every CTA is resident from the start
    int compute = num_sms() - args.ag_copy_ctas;
    if (compute > args.total_tiles) compute = args.total_tiles;
    if (compute <= 0) return 6006;
    grid = compute + args.ag_copy_ctas;
  }
  kern<<<grid, kGemmThreads, GemmSmem<BN>::kTotal, stream>>>(tmA, tmB, tmL, args);
  OB_CHECK_LAUNCH();
  return 0;
}

}  // namespace ob

using namespace ob;

// Dispatch on operand major-ness and tile width.
static int dispatch(int bn, int a_mn, int b_mn, const void* A, const void* B, const GemmArgs& g,
                    long long a_rows, long long a_cols, long long lda, long long b_rows,
                    long long b_cols, long long ldb, cudaStream_t s) {
#define OB_CASE(BN_, AM, BMj)                                                                   \
  if (bn == BN_ && a_mn == AM && b_mn == BMj)                                                   \
    return launch_gemm<BN_, AM != 0, BMj != 0>(A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, s);
  OB_CASE(256, 0, 0)
  OB_CASE(256, 0, 1)
  OB_CASE(256, 1, 1)
  OB_CASE(256, 1, 0)
  OB_CASE(128, 0, 0)
  OB_CASE(128, 0, 1)
  OB_CASE(128, 1, 1)
  OB_CASE(128, 1, 0)
#undef OB_CASE
  return 5000;
}

static int pick_bn(int M, int N) {
  // A 128x256 tile halves B traffic per flop; use 128 columns when the wide tile would
  // leave SMs idle or waste more than a quarter of its columns.
  long long t256 = (long long)((M + BM - 1) / BM) * ((N + 255) / 256);
  if (N <= 128) return 128;
  if (N % 256 != 0 && N % 256 <= 128 && N < 1024) return 128;
  if (t256 < 148) return 128;
  return 256;
}

extern "C" {

// Plain GEMM.  a_mn / b_mn: 0 = K-major ([M,K] / [N,K] row-major), 1 = MN-major
// ([K,M] / [K,N] row-major).  out_mode: 0 bf16, 1 fp32, 2 fp32 accumulate.
// residual (optional, bf16 [M,N] with pitch ldr) is added before the store.
int ob_gemm_bf16(const void* A, const void* B, void* C, const void* residual, int M, int N, int K,
                 long long lda, long long ldb, long long ldc, long long ldr, int a_mn, int b_mn,
                 int out_mode, int bn_override, const void* bias, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((lda & 7) || (ldb & 7)) return 6001;  // TMA needs 16-byte row pitches
  if ((((uintptr_t)A) & 15) || (((uintptr_t)B) & 15)) return 6002;
  int bn = bn_override ? bn_override : pick_bn(M, N);
  GemmArgs g = {};
  g.M = M; g.N = N; g.K = K; g.mode = 0;
  g.num_m_blocks = (M + BM - 1) / BM;
  g.num_n_blocks = (N + bn - 1) / bn;
  g.total_tiles = g.num_m_blocks * g.num_n_blocks;
  g.C = C; g.ldc = ldc; g.out_mode = out_mode;
  g.residual = (const bf16*)residual; g.ldr = ldr;
  g.bias = (const bf16*)bias;
  g.status = status;
  long long a_rows = a_mn ? K : M, a_cols = a_mn ? M : K;
  long long b_rows = b_mn ? K : N, b_cols = b_mn ? N : K;
  return dispatch(bn, a_mn, b_mn, A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, stream);
}

// GEMM whose fp32 output rows are spread over `world` GPUs: row block r of C lives at
// peer_ptrs[r] (rows_per_peer rows, pitch ldc) and receives the tile through
// red.global.add.v4.f32 over NVLink.  The destination must be zeroed (or hold the running
// sum) before any rank launches; completion is published by the caller's barrier.
int ob_gemm_bf16_peer_reduce(const void* A, const void* B, void* const* peer_ptrs, int world,
                             int rows_per_peer, int M, int N, int K, long long lda, long long ldb,
                             long long ldc, int a_mn, int b_mn, int bf16_out, int first_owner, int* status,
                             cudaStream_t stream) {
  if (world > kMaxPeers) return 6003;
  if ((lda & 7) || (ldb & 7)) return 6001;
  int bn = pick_bn(M, N);
  GemmArgs g = {};
  g.M = M; g.N = N; g.K = K; g.mode = 0;
  g.num_m_blocks = (M + BM - 1) / BM;
  if (first_owner > 0 && first_owner < world)
    g.m_rot = (int)(((long long)first_owner * rows_per_peer / BM) % g.num_m_blocks);
  g.num_n_blocks = (N + bn - 1) / bn;
  g.total_tiles = g.num_m_blocks * g.num_n_blocks;
  g.C = nullptr; g.ldc = ldc; g.out_mode = bf16_out >= 2 ? 5 : bf16_out ? 4 : 3;   // 2 + s: store into slab s
  g.peer_slot = bf16_out >= 2 ? bf16_out - 2 : 0;
  for (int i = 0; i < world; ++i) g.peer_ptr[i] = (float*)peer_ptrs[i];
  g.rows_per_peer = rows_per_peer;
  g.status = status;
  long long a_rows = a_mn ? K : M, a_cols = a_mn ? M : K;
  long long b_rows = b_mn ? K : N, b_cols = b_mn ? N : K;
  return dispatch(bn, a_mn, b_mn, A, B, g, a_rows, a_cols, lda, b_rows, b_cols, ldb, stream);
}

// Grouped GEMM over ragged row groups (mixture-of-experts forward and input gradient).
//   C[rows of group g, :N] = A[rows of group g, :K] * B_g^T
// group_offsets: device int[G+1], every entry a multiple of 128; rows beyond
// group_offsets[G] are ignored.  max_rows bounds the row count (allocation size of A/C).
// b_mn = 0: B is [G, N, K]; b_mn = 1: B is [G, K, N].
int ob_gemm_bf16_grouped(const void* A, const void* B, void* C, const int* group_offsets, int G,
                         int max_rows, int N, int K, long long lda, long long ldc, int b_mn,
                         int out_mode, int* status, cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if ((lda & 7) || (max_rows % BM)) return 6001;
  int bn = (N % 256 == 0 || N > 512) ? 256 : 128;
  GemmArgs g = {};
  g.M = max_rows; g.N = N; g.K = K; g.mode = 1;
  g.num_groups = G; g.group_offsets = group_offsets;
  g.b_group_rows = b_mn ? K : N;
  g.b_mn = b_mn;
  g.num_m_blocks = max_rows / BM;
  g.num_n_blocks = (N + bn - 1) / bn;
  g.total_tiles = g.num_m_blocks * g.num_n_blocks;
  g.C = C; g.ldc = ldc; g.out_mode = out_mode;
  g.status = status;
  long long b_rows = (long long)G * (b_mn ? K : N), b_cols = b_mn ? N : K;
  return dispatch(bn, 0, b_mn, A, B, g, max_rows, K, lda, b_rows, b_cols, b_cols, stream);
}

// Grouped weight gradient: dW_g[N, K] (+)= A[rows of g, :N]^T * B[rows of g, :K].
// A and B are row-major token matrices (MN-major operands); C is [G, N, K].
int ob_gemm_bf16_grouped_wgrad(const void* A, const void* B, void* C, const int* group_offsets,
                               int G, int max_rows, int N, int K, long long lda, long long ldb,
                               int out_mode, int* status, cudaStream_t stream) {
  if ((lda & 7) || (ldb & 7)) return 6001;
  int bn = (K % 256 == 0) ? 256 : 128;
  GemmArgs g = {};
  g.M = N; g.N = K; g.K = max_rows; g.mode = 2;
  g.num_groups = G; g.group_offsets = group_offsets;
  g.num_m_blocks = (N + BM - 1) / BM;
  g.num_n_blocks = (K + bn - 1) / bn;
  g.total_tiles = G * g.num_m_blocks * g.num_n_blocks;
  g.C = C; g.ldc = K; g.c_group_stride = (long long)N * K; g.out_mode = out_mode;
  g.status = status;
  return dispatch(bn, 1, 1, A, B, g, max_rows, N, lda, max_rows, K, ldb, stream);
}

// All-gather -> GEMM in one launch.  Both operands K-major: C[M,N] = A[M,K] B[N,K]^T (+ residual).
// side 1: A's rows are spread over `world` GPUs (rows_per_rank each, contiguous [rows, K] chunks at
// src_ptrs[r]); side 2: B's rows.  The gathered operand is assembled in `full` (this GPU's memory,
// [rows_per_rank * world, K] contiguous), which stays valid after the launch.  flags: `world`
// device counters owned by the caller that only grow; target = their common value before this
// call + copy_ctas.  Peers' chunks must be complete before any rank launches (caller's barrier).
int ob_gemm_bf16_ag(const void* other, void* full, void* const* src_ptrs, void* C, const void* residual, int M, int N,
                    int K, long long ldc, long long ldr, int out_mode, int side, int world, int rank,
                    int rows_per_rank, unsigned* flags, unsigned target, int copy_ctas, int* status,
                    cudaStream_t stream) {
  if (world > kMaxPeers || world <= 0 || copy_ctas <= 0 || copy_ctas > 32) return 6003;
  if (side != 1 && side != 2) return 6005;
  if (K & 7) return 6001;
  int bn = 256;
  if (side == 2 && rows_per_rank % 256) bn = 128;
  if (side == 1 ? (rows_per_rank % BM) : (rows_per_rank % bn)) return 6007;
  if ((long long)rows_per_rank * world != (side == 1 ? M : N)) return 6007;
  GemmArgs g = {};
  g.M = M; g.N = N; g.K = K; g.mode = 0;
  g.num_m_blocks = (M + BM - 1) / BM;
  g.num_n_blocks = (N + bn - 1) / bn;
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
  return dispatch(bn, 0, 0, A, B, g, M, K, K, N, K, K, stream);
}

}  // extern "C"
