// Shared pieces of the tcgen05 GEMM kernels: argument block, tile description, and the store of
// one 32-column slice of an accumulator row (bf16 / fp32 / fp32-accumulate / peer reduction).
#pragma once
#include "sm100_common.cuh"

namespace ob {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kStages = 4;
constexpr int kGemmThreads = 192;
constexpr int kMaxPeers = 8;

struct GemmArgs {
  int M, N, K;
  int mode;                  // 0 plain, 1 grouped rows, 2 grouped reduction
  int num_groups;
  const int* group_offsets;  // [G+1] device, multiples of 128
  int b_group_rows;          // rows per group in B's stacked 2-D view
  int b_mn;                  // B operand major-ness (needed for the grouped row offset)
  int num_m_blocks, num_n_blocks, total_tiles;
  void* C;
  long long ldc;
  long long c_group_stride;  // mode 2: elements between consecutive groups' outputs
  int out_mode;              // 0 bf16, 1 fp32 store, 2 fp32 accumulate, 3 fp32 peer red.add, 4 bf16 peer red.add,
                             // 5 bf16 peer store into the sender's slot of the owner's staging buffer
  const bf16* residual;
  long long ldr;
  const bf16* bias;          // optional [N]: added to every row before the store (bf16 / fp32 store modes)
  // Cross-entropy statistics (512 x 256 tile kernel, bf16 output): for every row and every
  // 256-column tile the maximum of the fp32 logits and the sum of exp(logit - maximum) go to
  // ce_stats[row * num_n_blocks + tile] and the fp32 logit of the row's target column to
  // ce_tgt[row], all taken from the accumulator before it is rounded to bf16.
  const int* ce_targets;
  float2* ce_stats;
  float* ce_tgt;
  // out_mode 3: rows [r*rows_per_peer, (r+1)*rows_per_peer) live on peer r at peer_ptr[r]
  float* peer_ptr[kMaxPeers];
  int rows_per_peer;
  // out_mode 5: the owner's staging buffer holds one [rows_per_peer, ldc] slab per sender; this
  // GEMM writes slab `peer_slot` (plain 16-byte stores over NVLink, no atomics); the owner sums
  // the slabs afterwards (two-phase reduce-scatter).
  int peer_slot;
  // peer output modes: the tile rows are walked starting m_rot blocks further on (wrapping), so that
  // the GPUs of a group, which run the same GEMM at the same time, each write to a different owner
  // at any moment instead of all converging on owner 0, then owner 1, ...
  int m_rot;
  // gather mode: ag_side 1 = rows of A, 2 = rows of B are assembled inside this launch
  int ag_side, ag_world, ag_rank, ag_copy_ctas;
  int ag_rows_per_rank;            // multiple of the tile extent on that side
  const void* ag_src[kMaxPeers];   // every rank's chunk (contiguous rows)
  void* ag_dst;                    // this GPU's full operand (what the tensor map covers)
  long long ag_chunk_bytes;
  uint32_t* ag_flags;              // [world] counters, only ever incremented
  uint32_t ag_target;              // value a chunk's counter has when the chunk is complete
  // CTA-pair kernels only.  raster_gm: tile rows that share one sweep over the tile columns.
  // k_splits > 1 (reducing output modes only): the reduction is cut into k_splits
  // slices of k_per_split elements; every (tile, slice) is one unit of work and its partial result
  // is added to C with vector reductions.
  int raster_gm, k_splits, k_per_split;
  int* status;
};

struct TileInfo {
  int a_row0;    // first row (K-major) / first column (MN-major) of the A tile
  int b_row0;    // same for B (K-major: already offset by the group)
  int b_k_off;   // MN-major B in grouped mode: row offset of the group's matrix
  int c_row0;    // first output row
  int c_col0;    // first output column
  int rows_valid, cols_valid;
  int k_begin, k_end;
  long long c_off;  // extra element offset into C (mode 2)
  bool valid;
};


// Store 32 (or fewer) consecutive columns of output row `grow`, held as fp32 bit patterns in v.
__device__ __forceinline__ void gemm_store_slice(const GemmArgs& p, long long c_off, long long grow, int col0,
                                                 int ncols, uint32_t (&v)[32]) {
            // debug build: the slice must lie inside the output (plain modes) / inside the owner's block
            if (!OB_DEBUG_CHECK(grow >= 0 && grow < p.M && col0 >= 0 && col0 + ncols <= p.N && ncols <= 32, p.status))
              return;
            if (p.bias) {
              for (int i = 0; i < ncols; ++i)
                v[i] = __float_as_uint(__uint_as_float(v[i]) + __bfloat162float(__ldg(p.bias + col0 + i)));
            }
            if (p.residual) {
              const bf16* rp = p.residual + grow * p.ldr + col0;
              if (ncols == 32 && ((((uintptr_t)rp) & 15) == 0)) {
  #pragma unroll
                for (int i = 0; i < 4; ++i) {
                  uint4 q = *reinterpret_cast<const uint4*>(rp + i * 8);
                  uint32_t w[4] = {q.x, q.y, q.z, q.w};
  #pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    float2 f = unpack_bf16(w[j]);
                    v[i * 8 + j * 2] = __float_as_uint(__uint_as_float(v[i * 8 + j * 2]) + f.x);
                    v[i * 8 + j * 2 + 1] =
                        __float_as_uint(__uint_as_float(v[i * 8 + j * 2 + 1]) + f.y);
                  }
                }
              } else {
                for (int i = 0; i < ncols; ++i)
                  v[i] = __float_as_uint(__uint_as_float(v[i]) + __bfloat162float(rp[i]));
              }
            }
            if (p.out_mode == 0) {
              bf16* cp = (bf16*)p.C + c_off + grow * p.ldc + col0;
              if (ncols == 32 && ((((uintptr_t)cp) & 15) == 0)) {
  #pragma unroll
                for (int i = 0; i < 4; ++i) {
                  uint4 q;
                  q.x = pack_bf16(__uint_as_float(v[i * 8 + 0]), __uint_as_float(v[i * 8 + 1]));
                  q.y = pack_bf16(__uint_as_float(v[i * 8 + 2]), __uint_as_float(v[i * 8 + 3]));
                  q.z = pack_bf16(__uint_as_float(v[i * 8 + 4]), __uint_as_float(v[i * 8 + 5]));
                  q.w = pack_bf16(__uint_as_float(v[i * 8 + 6]), __uint_as_float(v[i * 8 + 7]));
                  *reinterpret_cast<uint4*>(cp + i * 8) = q;
                }
              } else {
                for (int i = 0; i < ncols; ++i) cp[i] = __float2bfloat16(__uint_as_float(v[i]));
              }
            } else if (p.out_mode == 4) {
    // bf16 peer reduction: two columns per 32-bit reduction, eight per instruction
    const int owner = (int)(grow / p.rows_per_peer);
    const long long lrow = grow - (long long)owner * p.rows_per_peer;
    bf16* cp = reinterpret_cast<bf16*>(p.peer_ptr[owner]) + lrow * p.ldc + col0;
    if (ncols == 32 && ((((uintptr_t)cp) & 15) == 0)) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t q0 = pack_bf16(__uint_as_float(v[i * 8 + 0]), __uint_as_float(v[i * 8 + 1]));
        const uint32_t q1 = pack_bf16(__uint_as_float(v[i * 8 + 2]), __uint_as_float(v[i * 8 + 3]));
        const uint32_t q2 = pack_bf16(__uint_as_float(v[i * 8 + 4]), __uint_as_float(v[i * 8 + 5]));
        const uint32_t q3 = pack_bf16(__uint_as_float(v[i * 8 + 6]), __uint_as_float(v[i * 8 + 7]));
        asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(cp + i * 8), "r"(q0), "r"(q1),
                     "r"(q2), "r"(q3)
                     : "memory");
      }
    } else {
      for (int i = 0; i < ncols; ++i) atomicAdd(reinterpret_cast<__nv_bfloat16*>(cp + i), __float2bfloat16(__uint_as_float(v[i])));
    }
  } else if (p.out_mode == 5) {
    const int owner = (int)(grow / p.rows_per_peer);
    const long long lrow = grow - (long long)owner * p.rows_per_peer + (long long)p.peer_slot * p.rows_per_peer;
    bf16* cp = reinterpret_cast<bf16*>(p.peer_ptr[owner]) + lrow * p.ldc + col0;
    if (ncols == 32 && ((((uintptr_t)cp) & 15) == 0)) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 q;
        q.x = pack_bf16(__uint_as_float(v[i * 8 + 0]), __uint_as_float(v[i * 8 + 1]));
        q.y = pack_bf16(__uint_as_float(v[i * 8 + 2]), __uint_as_float(v[i * 8 + 3]));
        q.z = pack_bf16(__uint_as_float(v[i * 8 + 4]), __uint_as_float(v[i * 8 + 5]));
        q.w = pack_bf16(__uint_as_float(v[i * 8 + 6]), __uint_as_float(v[i * 8 + 7]));
        *reinterpret_cast<uint4*>(cp + i * 8) = q;
      }
    } else {
      for (int i = 0; i < ncols; ++i) cp[i] = __float2bfloat16(__uint_as_float(v[i]));
    }
  } else if (p.out_mode == 3) {
              const int owner = (int)(grow / p.rows_per_peer);
              const long long lrow = grow - (long long)owner * p.rows_per_peer;
              float* cp = p.peer_ptr[owner] + lrow * p.ldc + col0;
              if (ncols == 32 && ((((uintptr_t)cp) & 15) == 0)) {
  #pragma unroll
                for (int i = 0; i < 8; ++i) {
                  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp + i * 4),
                               "f"(__uint_as_float(v[i * 4 + 0])), "f"(__uint_as_float(v[i * 4 + 1])),
                               "f"(__uint_as_float(v[i * 4 + 2])), "f"(__uint_as_float(v[i * 4 + 3]))
                               : "memory");
                }
              } else {
                for (int i = 0; i < ncols; ++i) atomicAdd(cp + i, __uint_as_float(v[i]));
              }
            } else {
              float* cp = (float*)p.C + c_off + grow * p.ldc + col0;
              const bool accum = p.out_mode == 2;
              if (accum && p.k_splits > 1) {
                // several units add into the same tile: fire-and-forget vector reductions
                if (ncols == 32 && ((((uintptr_t)cp) & 15) == 0)) {
  #pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp + i * 4),
                                 "f"(__uint_as_float(v[i * 4 + 0])), "f"(__uint_as_float(v[i * 4 + 1])),
                                 "f"(__uint_as_float(v[i * 4 + 2])), "f"(__uint_as_float(v[i * 4 + 3]))
                                 : "memory");
                  }
                } else {
                  for (int i = 0; i < ncols; ++i) atomicAdd(cp + i, __uint_as_float(v[i]));
                }
              } else if (ncols == 32 && ((((uintptr_t)cp) & 15) == 0)) {
  #pragma unroll
                for (int i = 0; i < 8; ++i) {
                  float4 q = make_float4(__uint_as_float(v[i * 4 + 0]), __uint_as_float(v[i * 4 + 1]),
                                         __uint_as_float(v[i * 4 + 2]), __uint_as_float(v[i * 4 + 3]));
                  if (accum) {
                    float4 o = *reinterpret_cast<const float4*>(cp + i * 4);
                    q.x += o.x; q.y += o.y; q.z += o.z; q.w += o.w;
                  }
                  *reinterpret_cast<float4*>(cp + i * 4) = q;
                }
              } else {
                for (int i = 0; i < ncols; ++i)
                  cp[i] = __uint_as_float(v[i]) + (accum ? cp[i] : 0.f);
              }
            }
}

// Coalesced output of one 32-row x 32-column accumulator chunk to rows owned by other GPUs (output
// modes 3, 4, 5).  The accumulator arrives one row per lane, and a lane-per-row store sends 32
// separate 16-byte writes per instruction over NVLink (measured: 53 GB/s).  Here the chunk goes
// through a 4 KB shared-memory slab of the calling warp and leaves with the lanes laid along the
// row, so every instruction covers whole 128-byte (fp32) or 64-byte (bf16) row segments.
// `slab` must be 1024-byte aligned; all 32 lanes call (rows beyond M are masked inside).
__device__ __forceinline__ void peer_chunk_out(const GemmArgs& p, uint8_t* slab, int lane, long long grow0, int col0,
                                               const uint32_t (&v)[32]) {
  const uint32_t base = smem_u32(slab);
  if (p.out_mode == 3) {
    // fp32: 128 bytes per row, 16-byte chunk c of row r at r * 128 + ((c ^ (r & 7)) << 4)
#pragma unroll
    for (int c = 0; c < 8; ++c)
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + lane * 128 + (((uint32_t)c ^ (lane & 7)) << 4)),
                   "r"(v[c * 4 + 0]), "r"(v[c * 4 + 1]), "r"(v[c * 4 + 2]), "r"(v[c * 4 + 3])
                   : "memory");
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = it * 4 + (lane >> 3), c = lane & 7;
      uint32_t a, b, cc, d;
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(cc), "=r"(d)
                   : "r"(base + r * 128 + (((uint32_t)c ^ (r & 7)) << 4)));
      const long long grow = grow0 + r;
      if (grow < p.M) {
        const int owner = (int)(grow / p.rows_per_peer);
        float* cp = p.peer_ptr[owner] + (grow - (long long)owner * p.rows_per_peer) * p.ldc + col0 + c * 4;
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp), "f"(__uint_as_float(a)),
                     "f"(__uint_as_float(b)), "f"(__uint_as_float(cc)), "f"(__uint_as_float(d))
                     : "memory");
      }
    }
  } else {
    // bf16: 64 bytes per row, chunk c of row r at r * 64 + ((c ^ ((r >> 1) & 3)) << 4)
#pragma unroll
    for (int c = 0; c < 4; ++c)
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + lane * 64 + (((uint32_t)c ^ ((lane >> 1) & 3)) << 4)),
                   "r"(pack_bf16(__uint_as_float(v[c * 8 + 0]), __uint_as_float(v[c * 8 + 1]))),
                   "r"(pack_bf16(__uint_as_float(v[c * 8 + 2]), __uint_as_float(v[c * 8 + 3]))),
                   "r"(pack_bf16(__uint_as_float(v[c * 8 + 4]), __uint_as_float(v[c * 8 + 5]))),
                   "r"(pack_bf16(__uint_as_float(v[c * 8 + 6]), __uint_as_float(v[c * 8 + 7])))
                   : "memory");
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int r = it * 8 + (lane >> 2), c = lane & 3;
      uint32_t a, b, cc, d;
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(cc), "=r"(d)
                   : "r"(base + r * 64 + (((uint32_t)c ^ ((r >> 1) & 3)) << 4)));
      const long long grow = grow0 + r;
      if (grow < p.M) {
        const int owner = (int)(grow / p.rows_per_peer);
        long long lrow = grow - (long long)owner * p.rows_per_peer;
        if (p.out_mode == 5) lrow += (long long)p.peer_slot * p.rows_per_peer;
        bf16* cp = reinterpret_cast<bf16*>(p.peer_ptr[owner]) + lrow * p.ldc + col0 + c * 8;
        if (p.out_mode == 5) *reinterpret_cast<uint4*>(cp) = make_uint4(a, b, cc, d);
        else asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(cp), "r"(a), "r"(b), "r"(cc), "r"(d)
                          : "memory");
      }
    }
  }
  __syncwarp();   // the slab may be rewritten by the next chunk
}

// Gather-mode copy role (one thread): chunk by chunk, own chunk first, this CTA's share of every
// chunk travels owner -> shared-memory ring -> local full operand in 32 KB bulk copies.
// kRing 32 KB slots must fit below the barrier area of the launching kernel's shared memory.
template <int kRing>
__device__ __forceinline__ void ag_copy_role(const GemmArgs& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag) {
  constexpr int kPiece = 32768;
  static_assert(kRing >= 3 && kRing <= 6, "ring of 3 to 6 slots");
  constexpr int kLoads = kRing - 2;   // loads in flight; the other two slots may still be draining to memory
  for (int i = 0; i < kRing; ++i) mbar_init(&bars[i], 1);
  *abort_flag = 0;
  mbar_fence_init();
  const int W = p.ag_world, C = p.ag_copy_ctas, cta = blockIdx.x;
  const long long per = ((p.ag_chunk_bytes + C - 1) / C + 15) & ~15ll;
  const long long lo = (long long)cta * per;
  const long long hi = lo + per < p.ag_chunk_bytes ? lo + per : p.ag_chunk_bytes;
  const long long npc = hi > lo ? (hi - lo + kPiece - 1) / kPiece : 0;
  if (npc == 0) {
    for (int r = 0; r < W; ++r) red_release_gpu_add(p.ag_flags + r, 1);
    return;
  }
  const long long total = npc * W;
  long long head = 0, tail = 0;
  bool ok = true;
  while (tail < total && ok) {
    while (head < total && head - tail < kLoads) {
      // slot head % kRing was last read by store head - kRing; stores 0 .. tail-1 are committed, so at
      // most tail-1 - (head-kRing) >= kRing - kLoads of the newest ones may still be pending
      if (head >= kRing) tma_store_wait_read<kRing - kLoads>();
      const int r = (p.ag_rank + 1 + (int)(head / npc)) % W;   // own chunk last: nobody waits for it
      const long long off = lo + (head % npc) * kPiece;
      const uint32_t n = (uint32_t)(hi - off < kPiece ? hi - off : kPiece);
      const int slot = (int)(head % kRing);
      mbar_expect_tx(&bars[slot], n);
      bulk_g2s(smem + slot * kPiece, (const char*)p.ag_src[r] + off, n, &bars[slot]);
      ++head;
    }
    const int slot = (int)(tail % kRing);
    ok = mbar_wait(&bars[slot], (uint32_t)((tail / kRing) & 1), abort_flag, p.status, OB_ERR_WAIT_MISC);
    if (!ok) break;
    const int r = (p.ag_rank + 1 + (int)(tail / npc)) % W;
    const long long pi = tail % npc;
    const long long off = lo + pi * kPiece;
    const uint32_t n = (uint32_t)(hi - off < kPiece ? hi - off : kPiece);
    bulk_s2g((char*)p.ag_dst + (long long)r * p.ag_chunk_bytes + off, smem + slot * kPiece, n);
    tma_store_commit();
    if (pi == npc - 1) {  // this CTA's share of chunk r is in place
      tma_store_wait_all<0>();
      __threadfence();
      red_release_gpu_add(p.ag_flags + r, 1);
    }
    ++tail;
  }
  tma_store_wait_all<0>();
}

}  // namespace ob
