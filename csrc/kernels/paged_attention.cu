// Paged KV cache: append and single-token (decode) attention through a block table (page size 16 by default).
//
// Decode attention is bandwidth-bound (every cached key and value is read once per step), so the kernel is built
// around memory access and parallelism: one CTA per (sequence, KV head, 256-token slice of the context) serves all
// query heads of that group (split-KV, so a batch of 32 sequences still fills 148 SMs); K rows are fetched
// coalesced into a padded shared tile and scored with one lane per cached token, the weighted sum of values runs
// with one lane per slice of the head dimension (coalesced), and a second kernel merges the slices'
// (max, sum, output) triples.
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
constexpr int kSplitTokens = 256;          // cached tokens per CTA (split-KV): 2 passes of 32 tokens per warp

// Split-KV decode attention.  One CTA = (sequence, KV head, 256-token slice of the context); the slices of a sequence
// run on different SMs and a second kernel merges their (max, sum, accumulator) triples.  Inside a CTA a warp takes
// 32 tokens at a time: the K rows are fetched with fully coalesced 16-byte loads (16 lanes per 256-byte row) into a
// padded shared tile, then every lane scores ITS token against the group's query heads from shared memory; the value
// pass walks the tokens with all lanes on one coalesced V row.
template <int D>
__global__ void __launch_bounds__(kPaWarps * 32)
paged_decode_split_kernel(const __nv_bfloat16* __restrict__ q, long long ld_q, const __nv_bfloat16* __restrict__ k_cache,
                          const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_tables, int max_blocks,
                          const int* __restrict__ context_lens, int heads, int kv_heads, int block_size,
                          long long num_blocks, float scale, int g0, int gcount, float* __restrict__ partial, int nsplit) {
  constexpr int DL = D / 32;                 // head-dim elements per lane in the value pass
  constexpr int LPR = D / 8;                 // lanes per K row (16-byte pieces)
  constexpr int RPI = 32 / LPR;              // K rows fetched per warp instruction
  constexpr int KROW = D + 8;                // padded row (elements): 16-byte reads of 32 different rows hit 32 banks groups
  constexpr int kTileBytes = kPaWarps * 32 * KROW * 2;
  constexpr int kAccBytes = kPaWarps * kMaxGroup * D * 4;
  __shared__ __align__(16) uint8_t big[kTileBytes > kAccBytes ? kTileBytes : kAccBytes];   // K tiles, later the warp merge
  __shared__ float q_sh[kMaxGroup][D];
  __shared__ float m_sh[kPaWarps][kMaxGroup], l_sh[kPaWarps][kMaxGroup];
  const int b = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = heads / kv_heads;
  const int ctx = context_lens[b];
  const int t_begin = sp * kSplitTokens;
  if (t_begin >= ctx) return;
  const int t_end = min(ctx, t_begin + kSplitTokens);
  const int h_base = hk * group + g0;        // first query head of this pass
  __nv_bfloat16* k_tile = reinterpret_cast<__nv_bfloat16*>(big) + warp * 32 * KROW;

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

  const long long row = static_cast<long long>(kv_heads) * D;          // elements per cached token
  for (int base = t_begin + warp * 32; base < t_end; base += kPaWarps * 32) {
    const int tok = base + lane;
    const bool valid = tok < t_end;
    long long slot = 0;
    if (valid) {
      const int blk_idx = tok / block_size;
      int blk = blk_idx < max_blocks ? block_tables[static_cast<long long>(b) * max_blocks + blk_idx] : -1;
      if (blk < 0 || blk >= num_blocks) blk = 0;                     // corrupt tables read block 0 instead of faulting
      slot = static_cast<long long>(blk) * block_size + (tok - blk_idx * block_size);
    }
    const int n_tok = min(32, t_end - base);
    // ---- K rows of the 32 tokens -> shared tile (coalesced: LPR lanes per row)
    __syncwarp();
#pragma unroll
    for (int r0 = 0; r0 < 32; r0 += RPI) {
      const int r = r0 + lane / LPR;
      const long long slot_r = __shfl_sync(0xffffffffu, slot, r);
      if (r < n_tok) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(k_cache + slot_r * row + static_cast<long long>(hk) * D) + (lane % LPR));
        *reinterpret_cast<uint4*>(k_tile + r * KROW + (lane % LPR) * 8) = u;
      }
    }
    __syncwarp();
    // ---- scores: this lane's token against every query head of the group
    float s[kMaxGroup];
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) s[g] = 0.f;
    if (valid) {
      const __nv_bfloat16* kp = k_tile + lane * KROW;
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
    float p[kMaxGroup];
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) {
      if (g < gcount) {
        const float sv = valid ? s[g] : -INFINITY;
        const float mx = fmaxf(m[g], warp_max(sv));
        const float alpha = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mx);
        p[g] = valid ? __expf(sv - mx) : 0.f;
        l[g] = l[g] * alpha + warp_sum(p[g]);
        m[g] = mx;
#pragma unroll
        for (int j = 0; j < DL; ++j) acc[g][j] *= alpha;
      }
    }
    // ---- values: lanes own slices of the head dimension; two tokens' rows are in flight at a time
    for (int t = 0; t < n_tok; t += 2) {
      const bool two = t + 1 < n_tok;
      const long long slot_a = __shfl_sync(0xffffffffu, slot, t);
      const long long slot_b = __shfl_sync(0xffffffffu, slot, two ? t + 1 : t);
      const __nv_bfloat16* va = v_cache + slot_a * row + static_cast<long long>(hk) * D + lane * DL;
      const __nv_bfloat16* vb = v_cache + slot_b * row + static_cast<long long>(hk) * D + lane * DL;
      float v0[DL], v1[DL];
      if (DL == 4) {
        const uint2 ua = __ldg(reinterpret_cast<const uint2*>(va));
        const uint2 ub = __ldg(reinterpret_cast<const uint2*>(vb));
        const float2 a0 = unpack_bf16x2(ua.x), a1 = unpack_bf16x2(ua.y), b0 = unpack_bf16x2(ub.x), b1 = unpack_bf16x2(ub.y);
        v0[0] = a0.x; v0[1] = a0.y; v0[2] = a1.x; v0[3] = a1.y;
        v1[0] = b0.x; v1[1] = b0.y; v1[2] = b1.x; v1[3] = b1.y;
      } else {
        const float2 a0 = unpack_bf16x2(__ldg(reinterpret_cast<const uint32_t*>(va)));
        const float2 b0 = unpack_bf16x2(__ldg(reinterpret_cast<const uint32_t*>(vb)));
        v0[0] = a0.x; v0[1] = a0.y;
        v1[0] = b0.x; v1[1] = b0.y;
      }
#pragma unroll
      for (int g = 0; g < kMaxGroup; ++g) {
        if (g < gcount) {
          const float pa = __shfl_sync(0xffffffffu, p[g], t);
          const float pb = two ? __shfl_sync(0xffffffffu, p[g], t + 1) : 0.f;
#pragma unroll
          for (int j = 0; j < DL; ++j) acc[g][j] += pa * v0[j] + pb * v1[j];
        }
      }
    }
  }

  // ---- merge the warps, write this slice's (max, sum, accumulator) per head
  __syncthreads();                            // every warp is done with its K tile: the buffer becomes the merge area
  float (*acc_sh)[kMaxGroup][D] = reinterpret_cast<float (*)[kMaxGroup][D]>(big);
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
    float* pp = partial + ((static_cast<long long>(b) * heads + h_base + g) * nsplit + sp) * (D + 2);
    pp[2 + d] = num;
    if (d == 0) { pp[0] = mx; pp[1] = den; }
  }
}

// out[b, h, :] = merge over the slices that hold tokens of sequence b
template <int D>
__global__ void __launch_bounds__(D)
paged_decode_merge_kernel(const float* __restrict__ partial, const int* __restrict__ context_lens, int heads, int nsplit,
                          __nv_bfloat16* __restrict__ out, long long ld_o) {
  const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const int ctx = context_lens[b];
  const int n = min(nsplit, (ctx + kSplitTokens - 1) / kSplitTokens);
  const float* base = partial + (static_cast<long long>(b) * heads + h) * nsplit * (D + 2);
  float mx = -INFINITY;
  for (int s = 0; s < n; ++s) mx = fmaxf(mx, base[s * (D + 2)]);
  float num = 0.f, den = 0.f;
  for (int s = 0; s < n; ++s) {
    const float ms = base[s * (D + 2)];
    const float sc = (ms == -INFINITY) ? 0.f : __expf(ms - mx);
    num += base[s * (D + 2) + 2 + d] * sc;
    den += base[s * (D + 2) + 1] * sc;
  }
  out[static_cast<long long>(b) * ld_o + static_cast<long long>(h) * D + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
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

RB_API long long rb_paged_attention_scratch_floats(int batch, int heads, int head_dim, int max_blocks, int block_size) {
  const long long nsplit = (static_cast<long long>(max_blocks) * block_size + rb::kSplitTokens - 1) / rb::kSplitTokens;
  return static_cast<long long>(batch) * heads * nsplit * (head_dim + 2);
}

RB_API int rb_paged_attention_decode(const void* q, long long ld_q, void* out, long long ld_o, const void* k_cache,
                                     const void* v_cache, const int* block_tables, int max_blocks, const int* context_lens,
                                     int batch, int heads, int kv_heads, int head_dim, int block_size, long long num_blocks,
                                     float scale, float* scratch, void* stream_v) {
  if (batch <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || (head_dim != 64 && head_dim != 128) || block_size <= 0 ||
      max_blocks <= 0 || !scratch)
    return -1;
  if ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) return -2;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const int group = heads / kv_heads;
  const int nsplit = static_cast<int>((static_cast<long long>(max_blocks) * block_size + rb::kSplitTokens - 1) / rb::kSplitTokens);
  dim3 grid(batch, kv_heads, nsplit);
  auto Q = reinterpret_cast<const __nv_bfloat16*>(q);
  auto O = reinterpret_cast<__nv_bfloat16*>(out);
  auto K = reinterpret_cast<const __nv_bfloat16*>(k_cache);
  auto V = reinterpret_cast<const __nv_bfloat16*>(v_cache);
  for (int g0 = 0; g0 < group; g0 += rb::kMaxGroup) {     // groups wider than 8 heads take several passes
    const int gc = group - g0 < rb::kMaxGroup ? group - g0 : rb::kMaxGroup;
    if (head_dim == 128)
      rb::paged_decode_split_kernel<128><<<grid, rb::kPaWarps * 32, 0, stream>>>(Q, ld_q, K, V, block_tables, max_blocks,
                                                                                context_lens, heads, kv_heads, block_size,
                                                                                num_blocks, scale, g0, gc, scratch, nsplit);
    else
      rb::paged_decode_split_kernel<64><<<grid, rb::kPaWarps * 32, 0, stream>>>(Q, ld_q, K, V, block_tables, max_blocks,
                                                                               context_lens, heads, kv_heads, block_size,
                                                                               num_blocks, scale, g0, gc, scratch, nsplit);
  }
  dim3 mgrid(batch, heads);
  if (head_dim == 128)
    rb::paged_decode_merge_kernel<128><<<mgrid, 128, 0, stream>>>(scratch, context_lens, heads, nsplit, O, ld_o);
  else
    rb::paged_decode_merge_kernel<64><<<mgrid, 64, 0, stream>>>(scratch, context_lens, heads, nsplit, O, ld_o);
  return static_cast<int>(cudaGetLastError());
}
