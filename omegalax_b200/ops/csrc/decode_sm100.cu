// K8: decode-time attention over a paged KV cache.
//
// Cache layout: k_pages / v_pages [num_pages, page_size, G, HD] (bf16); block_table [B, max_blocks]
// maps the logical block j of sequence b to a physical page; seq_lens [B] counts the tokens
// already stored (padding never enters the cache, so every sequence has its own length).
//
//  decode_append_kernel   per new token: per-head RMSNorm of q and k (optional), rotate-half RoPE
//                         at the token's own position, q -> q_out, k and v -> their page slot.
//  decode_attn_kernel     one CTA per (sequence, kv head, KV split): the R = H/G query heads of
//                         the group share every K/V row that is read (GQA grouping), online
//                         softmax in fp32, partial (m, l, o) per split.
//  decode_combine_kernel  merges the splits.
// Decode is bound by reading the cache once, so these are CUDA-core kernels built around 16-byte
// loads; the tensor cores are not involved.
#include "host_utils.h"
#include "sm100_common.cuh"

namespace ob {

// one warp per (token, head) of the fused [q heads | k heads | v heads] projection
template <bool kOnePlus>
__global__ void decode_append_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ qw,
                                     const bf16* __restrict__ kw, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token, const int* __restrict__ slot_of_token,
                                     const int* __restrict__ block_table, int max_blocks, int page_size,
                                     bf16* __restrict__ q_out, bf16* __restrict__ k_pages,
                                     bf16* __restrict__ v_pages, long long ntok, int H, int G, int HD, int rot,
                                     float theta, float eps) {
  const int lane = threadIdx.x & 31;
  const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int HH = H + 2 * G;
  if (wid >= ntok * HH) return;
  const long long t = wid / HH;
  const int h = (int)(wid - t * HH);
  const bf16* src = qkv + t * (long long)HH * HD + (long long)h * HD;
  const int b = seq_of_token[t];
  const int slot = slot_of_token[t];                 // index of this token inside its sequence
  const int page = block_table[(long long)b * max_blocks + slot / page_size];
  const long long cache_row = ((long long)page * page_size + slot % page_size) * G;
  if (h >= H + G) {                                   // value head: plain copy
    bf16* dst = v_pages + (cache_row + (h - H - G)) * HD;
    for (int i = lane; i < HD; i += 32) dst[i] = src[i];
    return;
  }
  const bool is_q = h < H;
  const bf16* w = is_q ? qw : kw;
  bf16* dst = is_q ? q_out + (t * H + h) * HD : k_pages + (cache_row + (h - H)) * HD;
  float ss = 0.f;
  for (int i = lane; i < HD; i += 32) {
    float v = __bfloat162float(src[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float rstd = w ? rsqrtf(ss / (float)HD + eps) : 1.f;
  const int half = rot >> 1;
  const float pos = (float)positions[t];
  for (int i = lane; i < half; i += 32) {
    float w1 = 1.f, w2 = 1.f;
    if (w) {
      w1 = __bfloat162float(w[i]) + (kOnePlus ? 1.f : 0.f);
      w2 = __bfloat162float(w[i + half]) + (kOnePlus ? 1.f : 0.f);
    }
    float x1 = __bfloat162float(__float2bfloat16(__bfloat162float(src[i]) * rstd * w1));
    float x2 = __bfloat162float(__float2bfloat16(__bfloat162float(src[i + half]) * rstd * w2));
    float inv = __powf(theta, -(float)(2 * i) / (float)rot);
    float s, c;
    sincosf(pos * inv, &s, &c);
    dst[i] = __float2bfloat16(x1 * c - x2 * s);
    dst[i + half] = __float2bfloat16(x2 * c + x1 * s);
  }
  for (int i = rot + lane; i < HD; i += 32) {
    float wv = w ? __bfloat162float(w[i]) + (kOnePlus ? 1.f : 0.f) : 1.f;
    dst[i] = __float2bfloat16(__bfloat162float(src[i]) * rstd * wv);
  }
}

// grid (B, G, splits); 128 threads = 8 half-warps; half-warp w walks keys w, w+8, ... of the split.
// HD = 128: each lane owns 8 consecutive channels (one 16-byte load per K and V row).
// R <= 8 query heads per kv head share every row that is read.
template <int HD, int R>
__global__ void __launch_bounds__(128)
decode_attn_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                   const int* __restrict__ block_table, const int* __restrict__ seq_lens, int max_blocks,
                   int page_size, int G, int splits, float scale, float* __restrict__ part_o,
                   float* __restrict__ part_ml) {
  static_assert(HD == 128, "one half-warp covers a 128-channel row");
  constexpr int C = 8;    // channels per lane
  constexpr int NW = 8;   // half-warps per CTA
  const int b = blockIdx.x, g = blockIdx.y, sp = blockIdx.z;
  const int sub = threadIdx.x >> 4, hl = threadIdx.x & 15;
  const int H = G * R;
  const int S = seq_lens[b];
  const int per = (S + splits - 1) / splits;
  const int k_lo = sp * per, k_hi = min(S, k_lo + per);
  float qv[R][C];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint4 u = *reinterpret_cast<const uint4*>(q + ((long long)b * H + g * R + r) * HD + hl * C);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float2 t = unpack_bf16(w[c]);
      qv[r][2 * c] = t.x * scale; qv[r][2 * c + 1] = t.y * scale;
    }
  }
  float m[R], l[R], o[R][C];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < C; ++c) o[r][c] = 0.f;
  }
  // Four key rows per half-warp and iteration: the block-table lookups and the eight 16-byte row
  // loads of an iteration are issued back to back before any arithmetic, so a thread keeps 128
  // bytes in flight (the kernel is latency bound otherwise: one K and one V row per round trip).
  constexpr int U = 4;
  for (int s0 = k_lo; s0 < k_hi; s0 += NW * U) {   // uniform trip count: the shuffles below need all lanes
    uint4 ku[U], vu[U];
    bool okv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int s = s0 + u * NW + sub;
      okv[u] = s < k_hi;
      ku[u] = make_uint4(0, 0, 0, 0);
      vu[u] = make_uint4(0, 0, 0, 0);
      if (okv[u]) {
        const int page = __ldg(block_table + (long long)b * max_blocks + s / page_size);
        const long long row = (((long long)page * page_size + s % page_size) * G + g) * HD + hl * C;
        ku[u] = *reinterpret_cast<const uint4*>(k_pages + row);
        vu[u] = *reinterpret_cast<const uint4*>(v_pages + row);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool ok = okv[u];
      float kv[C], vv[C];
      const uint32_t kw[4] = {ku[u].x, ku[u].y, ku[u].z, ku[u].w}, vw[4] = {vu[u].x, vu[u].y, vu[u].z, vu[u].w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float2 a = unpack_bf16(kw[c]), d = unpack_bf16(vw[c]);
        kv[2 * c] = a.x; kv[2 * c + 1] = a.y;
        vv[2 * c] = d.x; vv[2 * c + 1] = d.y;
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float d = 0.f;
#pragma unroll
        for (int c = 0; c < C; ++c) d = fmaf(qv[r][c], kv[c], d);
#pragma unroll
        for (int x = 8; x > 0; x >>= 1) d += __shfl_xor_sync(0xffffffffu, d, x);
        if (ok) {
          const float mn = fmaxf(m[r], d);
          const float a = __expf(m[r] - mn), p = __expf(d - mn);
          l[r] = l[r] * a + p;
#pragma unroll
          for (int c = 0; c < C; ++c) o[r][c] = o[r][c] * a + p * vv[c];
          m[r] = mn;
        }
      }
    }
  }
  // merge the eight half-warps through shared memory
  __shared__ float sm_m[NW][R], sm_l[NW][R], sm_o[NW][R][HD];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (hl == 0) { sm_m[sub][r] = m[r]; sm_l[sub][r] = l[r]; }
#pragma unroll
    for (int c = 0; c < C; ++c) sm_o[sub][r][hl * C + c] = o[r][c];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < R * HD; idx += 128) {
    const int r = idx / HD, c = idx - r * HD;
    float mm = -INFINITY;
    for (int w = 0; w < NW; ++w) mm = fmaxf(mm, sm_m[w][r]);
    float ll = 0.f, oo = 0.f;
    for (int w = 0; w < NW; ++w) {
      const float a = (sm_m[w][r] == -INFINITY) ? 0.f : __expf(sm_m[w][r] - mm);
      ll += sm_l[w][r] * a;
      oo += sm_o[w][r][c] * a;
    }
    const long long base = (((long long)b * H + g * R + r) * splits + sp);
    part_o[base * HD + c] = oo;
    if (c == 0) { part_ml[base * 2] = mm; part_ml[base * 2 + 1] = ll; }
  }
}

__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      bf16* __restrict__ out, int splits, int HD) {
  const long long bh = blockIdx.x;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(bh * splits + s) * 2]);
  float ll = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(bh * splits + s) * 2];
    ll += (ms == -INFINITY) ? 0.f : part_ml[(bh * splits + s) * 2 + 1] * __expf(ms - mm);
  }
  for (int c = threadIdx.x; c < HD; c += blockDim.x) {
    float oo = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = part_ml[(bh * splits + s) * 2];
      if (ms != -INFINITY) oo += part_o[(bh * splits + s) * HD + c] * __expf(ms - mm);
    }
    out[bh * HD + c] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
  }
}

}  // namespace ob

using namespace ob;

extern "C" {

int ob_decode_append(const void* qkv, const void* qw, const void* kw, const int* positions,
                     const int* seq_of_token, const int* slot_of_token, const int* block_table, int max_blocks,
                     int page_size, void* q_out, void* k_pages, void* v_pages, long long ntok, int H, int G,
                     int HD, int rot, float theta, float eps, int one_plus, cudaStream_t s) {
  if (ntok <= 0) return 0;
  long long warps = ntok * (H + 2 * G);
  long long blocks = (warps * 32 + 255) / 256;
  if (one_plus)
    decode_append_kernel<true><<<(unsigned)blocks, 256, 0, s>>>(
        (const bf16*)qkv, (const bf16*)qw, (const bf16*)kw, positions, seq_of_token, slot_of_token, block_table,
        max_blocks, page_size, (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, ntok, H, G, HD, rot, theta, eps);
  else
    decode_append_kernel<false><<<(unsigned)blocks, 256, 0, s>>>(
        (const bf16*)qkv, (const bf16*)qw, (const bf16*)kw, positions, seq_of_token, slot_of_token, block_table,
        max_blocks, page_size, (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, ntok, H, G, HD, rot, theta, eps);
  OB_CHECK_LAUNCH();
  return 0;
}

// q [B,H,HD] -> out [B,H,HD]; part_o fp32 [B*H*splits*HD], part_ml fp32 [B*H*splits*2] scratch.
int ob_decode_attn(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                   const int* seq_lens, int B, int H, int G, int HD, int max_blocks, int page_size, int splits,
                   float scale, float* part_o, float* part_ml, void* out, cudaStream_t s) {
  if (B <= 0) return 0;
  if (HD != 128 || H % G) return 6005;
  const int R = H / G;
  dim3 grid(B, G, splits);
#define OB_DA(RR)                                                                                         \
  decode_attn_kernel<128, RR><<<grid, 128, 0, s>>>((const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, \
                                                    block_table, seq_lens, max_blocks, page_size, G, splits,   \
                                                    scale, part_o, part_ml)
  if (R == 1) OB_DA(1); else if (R == 2) OB_DA(2); else if (R == 4) OB_DA(4); else if (R == 8) OB_DA(8);
  else return 6005;
#undef OB_DA
  OB_CHECK_LAUNCH();
  decode_combine_kernel<<<(unsigned)(B * H), 128, 0, s>>>(part_o, part_ml, (bf16*)out, splits, HD);
  OB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
