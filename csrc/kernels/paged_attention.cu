// Paged KV cache: append and single-token (decode) attention through a block table (page size 16 by default).
//
// Decode attention is bandwidth-bound (every cached key and value is read once per step), so the kernel is built
// around memory access: one CTA per (sequence, KV head) serves all query heads of that group, four warps walk
// the sequence's pages two at a time; scores are computed with one lane per cached token, the weighted sum of
// values with one lane per slice of the head dimension (coalesced), and the four partial (max, sum, output)
// triples are merged at the end.
//
// The reference's PagedCache is block-table bookkeeping without tensor storage and its KVCache::append drops
// the new entries (crates/nn/src/kv_cache.rs:172-216,382-432); this is the storage and the kernel they lack.
#include "paged_attention.h"

#include <float.h>

#include "rb_common.cuh"

namespace rb {

__global__ void __launch_bounds__(128)
kv_append_kernel(const __nv_bfloat16* __restrict__ k_new, long long ld_k, const __nv_bfloat16* __restrict__ v_new,
                 long long ld_v, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                 const long long* __restrict__ slots, long long tokens, int row_elems, long long num_slots) {
  const int chunks = row_elems / 8;
  const long long total = tokens * chunks;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long t = i / chunks;
    const int c = static_cast<int>(i - t * chunks) * 8;
    const long long slot = slots[t];
    if (slot < 0 || slot >= num_slots) continue;
    *reinterpret_cast<uint4*>(k_cache + slot * row_elems + c) = *reinterpret_cast<const uint4*>(k_new + t * ld_k + c);
    *reinterpret_cast<uint4*>(v_cache + slot * row_elems + c) = *reinterpret_cast<const uint4*>(v_new + t * ld_v + c);
  }
}

constexpr int kMaxGroup = 8;     // query heads per KV head served by one CTA pass
constexpr int kPaWarps = 4;

template <int D>
__global__ void __launch_bounds__(kPaWarps * 32)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, long long ld_q, __nv_bfloat16* __restrict__ out, long long ld_o,
                    const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                    const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ context_lens,
                    int heads, int kv_heads, int block_size, long long num_blocks, float scale, int g0, int gcount) {
  constexpr int DL = D / 32;                 // head-dim elements per lane in the value pass
  __shared__ float q_sh[kMaxGroup][D];
  __shared__ float m_sh[kPaWarps][kMaxGroup], l_sh[kPaWarps][kMaxGroup];
  __shared__ float acc_sh[kPaWarps][kMaxGroup][D];
  const int b = blockIdx.x, hk = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = heads / kv_heads;
  const int ctx = context_lens[b];
  const int h_base = hk * group + g0;        // first query head of this pass

  for (int i = threadIdx.x; i < gcount * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    q_sh[g][d] = __bfloat162float(q[static_cast<long long>(b) * ld_q + static_cast<long long>(h_base + g) * D + d]) * scale;
  }
  __syncthreads();

  float m[kMaxGroup], l[kMaxGroup], acc[kMaxGroup][DL];
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DL; ++j) acc[g][j] = 0.f;
  }

  const int tokens_per_pass = 32;            // one lane per cached token
  const long long row = static_cast<long long>(kv_heads) * D;          // elements per cached token
  const int n_pass = (ctx + tokens_per_pass - 1) / tokens_per_pass;
  for (int pass = warp; pass < n_pass; pass += kPaWarps) {
    const int tok = pass * tokens_per_pass + lane;
    const bool valid = tok < ctx;
    long long slot = 0;
    if (valid) {
      const int blk_idx = tok / block_size;
      int blk = blk_idx < max_blocks ? block_tables[static_cast<long long>(b) * max_blocks + blk_idx] : -1;
      if (blk < 0 || blk >= num_blocks) blk = 0;                     // corrupt tables read block 0 instead of faulting
      slot = static_cast<long long>(blk) * block_size + (tok - blk_idx * block_size);
    }
    // ---- scores: this lane's token against every query head of the group
    float s[kMaxGroup];
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) s[g] = 0.f;
    if (valid) {
      const __nv_bfloat16* kp = k_cache + slot * row + static_cast<long long>(hk) * D;
#pragma unroll 4
      for (int c = 0; c < D; c += 8) {
        const uint4 u = *reinterpret_cast<const uint4*>(kp + c);
        const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
          if (g < gcount) {
            const float* qq = &q_sh[g][c];
            s[g] += qq[0] * f0.x + qq[1] * f0.y + qq[2] * f1.x + qq[3] * f1.y + qq[4] * f2.x + qq[5] * f2.y +
                    qq[6] * f3.x + qq[7] * f3.y;
          }
        }
      }
    }
    // ---- online softmax over the 32 tokens of this pass
    float p[kMaxGroup], alpha[kMaxGroup];
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) {
      if (g < gcount) {
        const float sv = valid ? s[g] : -INFINITY;
        const float mx = fmaxf(m[g], warp_max(sv));
        alpha[g] = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mx);
        p[g] = valid ? __expf(sv - mx) : 0.f;
        l[g] = l[g] * alpha[g] + warp_sum(p[g]);
        m[g] = mx;
#pragma unroll
        for (int j = 0; j < DL; ++j) acc[g][j] *= alpha[g];
      }
    }
    // ---- values: lanes own slices of the head dimension, tokens are visited one by one
    const int n_tok = min(tokens_per_pass, ctx - pass * tokens_per_pass);
    for (int t = 0; t < n_tok; ++t) {
      const long long slot_t = __shfl_sync(0xffffffffu, slot, t);
      const __nv_bfloat16* vp = v_cache + slot_t * row + static_cast<long long>(hk) * D + lane * DL;
      float v[DL];
      if (DL == 4) {
        const uint2 u = *reinterpret_cast<const uint2*>(vp);
        const float2 a = unpack_bf16x2(u.x), c2 = unpack_bf16x2(u.y);
        v[0] = a.x; v[1] = a.y; v[2] = c2.x; v[3] = c2.y;
      } else {
        const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(vp));
        v[0] = a.x; v[1] = a.y;
      }
#pragma unroll
      for (int g = 0; g < kMaxGroup; ++g) {
        if (g < gcount) {
          const float pt = __shfl_sync(0xffffffffu, p[g], t);
#pragma unroll
          for (int j = 0; j < DL; ++j) acc[g][j] += pt * v[j];
        }
      }
    }
  }

  // ---- merge the warps
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) {
    if (g < gcount) {
      if (lane == 0) { m_sh[warp][g] = m[g]; l_sh[warp][g] = l[g]; }
#pragma unroll
      for (int j = 0; j < DL; ++j) acc_sh[warp][g][lane * DL + j] = acc[g][j];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < gcount * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < kPaWarps; ++w) mx = fmaxf(mx, m_sh[w][g]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < kPaWarps; ++w) {
      const float sc = (m_sh[w][g] == -INFINITY) ? 0.f : __expf(m_sh[w][g] - mx);
      num += acc_sh[w][g][d] * sc;
      den += l_sh[w][g] * sc;
    }
    out[static_cast<long long>(b) * ld_o + static_cast<long long>(h_base + g) * D + d] =
        __float2bfloat16(den > 0.f ? num / den : 0.f);
  }
}

}  // namespace rb

RB_API int rb_kv_append(const void* k_new, long long ld_k, const void* v_new, long long ld_v, void* k_cache, void* v_cache,
                        const long long* slot_mapping, long long tokens, int kv_heads, int head_dim, long long num_slots,
                        void* stream_v) {
  if (tokens <= 0) return 0;
  const int row = kv_heads * head_dim;
  if (row <= 0 || (row % 8) || (ld_k % 8) || (ld_v % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new) | reinterpret_cast<uintptr_t>(k_cache) |
       reinterpret_cast<uintptr_t>(v_cache)) & 15)
    return -2;
  const long long total = tokens * (row / 8);
  long long blocks = (total + 127) / 128;
  if (blocks > 148 * 16) blocks = 148 * 16;
  rb::kv_append_kernel<<<static_cast<int>(blocks), 128, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const __nv_bfloat16*>(k_new), ld_k, reinterpret_cast<const __nv_bfloat16*>(v_new), ld_v,
      reinterpret_cast<__nv_bfloat16*>(k_cache), reinterpret_cast<__nv_bfloat16*>(v_cache), slot_mapping, tokens, row,
      num_slots);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_paged_attention_decode(const void* q, long long ld_q, void* out, long long ld_o, const void* k_cache,
                                     const void* v_cache, const int* block_tables, int max_blocks, const int* context_lens,
                                     int batch, int heads, int kv_heads, int head_dim, int block_size, long long num_blocks,
                                     float scale, void* stream_v) {
  if (batch <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || (head_dim != 64 && head_dim != 128) || block_size <= 0 ||
      max_blocks <= 0)
    return -1;
  if ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) return -2;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const int group = heads / kv_heads;
  dim3 grid(batch, kv_heads);
  for (int g0 = 0; g0 < group; g0 += rb::kMaxGroup) {     // groups wider than 8 heads take several passes
    const int gc = group - g0 < rb::kMaxGroup ? group - g0 : rb::kMaxGroup;
    auto Q = reinterpret_cast<const __nv_bfloat16*>(q);
    auto O = reinterpret_cast<__nv_bfloat16*>(out);
    auto K = reinterpret_cast<const __nv_bfloat16*>(k_cache);
    auto V = reinterpret_cast<const __nv_bfloat16*>(v_cache);
    if (head_dim == 128)
      rb::paged_decode_kernel<128><<<grid, rb::kPaWarps * 32, 0, stream>>>(Q, ld_q, O, ld_o, K, V, block_tables, max_blocks,
                                                                          context_lens, heads, kv_heads, block_size,
                                                                          num_blocks, scale, g0, gc);
    else
      rb::paged_decode_kernel<64><<<grid, rb::kPaWarps * 32, 0, stream>>>(Q, ld_q, O, ld_o, K, V, block_tables, max_blocks,
                                                                         context_lens, heads, kv_heads, block_size,
                                                                         num_blocks, scale, g0, gc);
  }
  return static_cast<int>(cudaGetLastError());
}
