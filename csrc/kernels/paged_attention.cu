// Paged KV cache: append and single-token (decode) attention through a block table (page size 16 by default).
//
// Decode attention is bandwidth-bound (every cached key and value is read once per step), so the kernel is built
// around memory access and parallelism: one CTA per (sequence, KV head, 256-token slice of the context) serves all
// query heads of that group (split-KV, so a batch of 32 sequences still fills 148 SMs); K and V rows are fetched
// coalesced into a padded shared tile, the group's heads are the rows of mma.sync tensor-core tiles for both
// Q K^T and P V, and a second kernel merges the slices' (max, sum, output) triples.
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
                 const long long* __restrict__ slots, long long tokens, int row_elems, long long num_slots RB_BOUNDS_PARAM) {
  const int chunks = row_elems / 8;
  const long long total = tokens * chunks;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long t = i / chunks;
    const int c = static_cast<int>(i - t * chunks) * 8;
    const long long slot = slots[t];
    if (slot >= num_slots && c == 0) RB_BOUNDS_HIT(103);           // a negative slot means "skip this token"
    if (slot < 0 || slot >= num_slots) continue;
    *reinterpret_cast<uint4*>(k_cache + slot * row_elems + c) = *reinterpret_cast<const uint4*>(k_new + t * ld_k + c);
    *reinterpret_cast<uint4*>(v_cache + slot * row_elems + c) = *reinterpret_cast<const uint4*>(v_new + t * ld_v + c);
  }
}

constexpr int kMaxGroup = 16;    // query heads per KV head served by one CTA pass (the M of the mma tile)
constexpr int kPaWarps = 4;
constexpr int kSplitTokens = 256;          // cached tokens per CTA (split-KV): 2 passes of 32 tokens per warp

__device__ __forceinline__ void pa_ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pa_ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pa_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16-byte asynchronous global -> shared copy; bytes == 0 writes zeros and reads nothing
__device__ __forceinline__ void pa_cp_async16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pa_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void pa_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t pa_pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Split-KV decode attention.  One CTA = (sequence, KV head, 256-token slice of the context); the slices of a sequence
// run on different SMs and a second kernel merges their (max, sum, accumulator) triples.  Inside a CTA a warp takes
// 32 tokens at a time.  Their K rows and V rows are fetched with fully coalesced 16-byte asynchronous copies (cp.async,
// 16 lanes per 256-byte row) into two padded shared tiles per warp; the K tile of the next pass is requested as soon
// as the scores of this pass are computed and the V tile as soon as P V is done, so every warp always has a tile in
// flight while it computes.  The query heads of the group
// form the 16 rows of an m16n8k16 tensor-core tile (rows beyond the group are zero): S = Q K^T is 4 n-tiles x D/16
// k-steps of mma.sync, the softmax runs on the accumulator fragments, and O += P V reuses those fragments as the A
// operand against ldmatrix.trans-fed V.  One query token per sequence gives M <= 16, far below the 64-row minimum
// of a tcgen05 tile, which is why this kernel is on the warp-level tensor path; it is bound by the K / V reads.
template <int D>
__global__ void __launch_bounds__(kPaWarps * 32, 3)
paged_decode_split_kernel(const __nv_bfloat16* __restrict__ q, long long ld_q, const __nv_bfloat16* __restrict__ k_cache,
                          const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_tables, int max_blocks,
                          const int* __restrict__ context_lens, int heads, int kv_heads, int block_size,
                          long long num_blocks, float scale, int g0, int gcount, float* __restrict__ partial, int nsplit
                          RB_BOUNDS_PARAM) {
  constexpr int LPR = D / 8;                 // lanes per K / V row (16-byte pieces)
  constexpr int RPI = 32 / LPR;              // rows fetched per warp instruction
  constexpr int NLD = 32 / RPI;              // load instructions per 32-row tile
  constexpr int KROW = D + 8;                // padded row (elements): ldmatrix rows 272 (144) bytes apart hit distinct banks
  constexpr int NT = D / 8;                  // n-tiles of the output accumulator
  constexpr int kTileElems = 32 * KROW;      // one K or V tile of one warp
  extern __shared__ __align__(16) uint8_t big[];   // [warp][K tile, V tile] bf16, then q_sh; later the warp merge area
  __nv_bfloat16* q_sh = reinterpret_cast<__nv_bfloat16*>(big) + kPaWarps * 2 * kTileElems;
  __shared__ float m_sh[kPaWarps][kMaxGroup], l_sh[kPaWarps][kMaxGroup];
  const int b = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, tq = lane & 3;   // fragment coordinates: row (and row + 8), column pair
  const int group = heads / kv_heads;
  const int ctx = context_lens[b];
  const int t_begin = sp * kSplitTokens;
  if (t_begin >= ctx) return;
  const int t_end = min(ctx, t_begin + kSplitTokens);
  const int h_base = hk * group + g0;        // first query head of this pass
  const uint32_t kt_u32 = smem_u32(reinterpret_cast<__nv_bfloat16*>(big) + warp * 2 * kTileElems);
  const uint32_t vt_u32 = kt_u32 + kTileElems * 2;
  const uint32_t q_u32 = smem_u32(q_sh);

  // the group's query rows as bf16 [16][D] (rows >= gcount are zero)
  for (int i = threadIdx.x; i < kMaxGroup * LPR; i += blockDim.x) {
    const int g = i / LPR, c = (i - g * LPR) * 8;
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (g < gcount) {
      const __nv_bfloat16* src = q + static_cast<long long>(b) * ld_q + static_cast<long long>(h_base + g) * D + c;
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = *reinterpret_cast<const uint32_t*>(src + 2 * j);   // rows are 4-byte aligned at least
      u = make_uint4(w[0], w[1], w[2], w[3]);
    }
    *reinterpret_cast<uint4*>(q_sh + g * KROW + c) = u;
  }
  __syncthreads();

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows gq and gq + 8
  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;

  const long long row = static_cast<long long>(kv_heads) * D;          // elements per cached token
  const int piece = (lane % LPR) * 8;
  const long long col = static_cast<long long>(hk) * D + piece;
  const uint32_t dst_off = ((lane / LPR) * KROW + piece) * 2;          // byte offset of this lane's piece in a tile
  int srow[NLD];                                                       // cache slot of the row behind each copy (-1: none)
  int n_next = 0;
  // cache slots of the 32 tokens that start at `first` (the host bounds num_blocks * block_size below 2^31)
  auto locate = [&](int first) {
    const int tok = first + lane;
    int slot = 0;
    if (tok < t_end) {
      const int blk_idx = tok / block_size;
      int blk = blk_idx < max_blocks ? block_tables[static_cast<long long>(b) * max_blocks + blk_idx] : -1;
      if (blk < 0 || blk >= num_blocks) {                            // corrupt tables read block 0 instead of faulting
        RB_BOUNDS_HIT(104);
        blk = 0;
      }
      slot = blk * block_size + (tok - blk_idx * block_size);
    }
    n_next = min(32, t_end - first);
#pragma unroll
    for (int i = 0; i < NLD; ++i) {
      const int r = i * RPI + lane / LPR;
      const int slot_r = __shfl_sync(0xffffffffu, slot, r);
      srow[i] = r < n_next ? slot_r : -1;
    }
  };
  // one tile = NLD asynchronous 16-byte copies per lane, one commit group; rows past the context are zero-filled
  auto request = [&](const __nv_bfloat16* cache, uint32_t tile_u32) {
#pragma unroll
    for (int i = 0; i < NLD; ++i) {
      const bool ok = srow[i] >= 0;
      pa_cp_async16(tile_u32 + dst_off + i * RPI * KROW * 2, ok ? cache + srow[i] * row + col : cache, ok ? 16 : 0);
    }
    pa_cp_commit();
  };
  int base = t_begin + warp * 32;
  if (base < t_end) {
    locate(base);
    request(k_cache, kt_u32);
    request(v_cache, vt_u32);
  }
  for (; base < t_end; base += kPaWarps * 32) {
    const int n_tok = n_next;
    const bool more = base + kPaWarps * 32 < t_end;
    pa_cp_wait<1>();                                                 // this pass's K tile has landed (V may be in flight)
    __syncwarp();
    // ---- S[16 heads, 32 tokens] = Q K^T
    float s[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16) {
      uint32_t a[4];
      // A fragment: matrices (rows 0-7, k0), (rows 8-15, k0), (rows 0-7, k0 + 8), (rows 8-15, k0 + 8)
      pa_ldsm_x4(q_u32 + ((lane & 15) * KROW + k0 + (lane >> 4) * 8) * 2, a);
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t bfr[4];
        // B fragments of two n-tiles: (tokens 16np..+7, k0), (same tokens, k0 + 8), (tokens 16np + 8.., k0), (.., k0 + 8)
        pa_ldsm_x4(kt_u32 + ((np * 16 + (lane & 7) + ((lane >> 4) << 3)) * KROW + k0 + ((lane >> 3) & 1) * 8) * 2, bfr);
        pa_mma(s[2 * np], a, bfr[0], bfr[1]);
        pa_mma(s[2 * np + 1], a, bfr[2], bfr[3]);
      }
    }
    __syncwarp();                                                    // every lane has read its K fragments
    if (more) {                                                      // the next pass's K tile flies under softmax and P V
      locate(base + kPaWarps * 32);
      request(k_cache, kt_u32);
    }
    // ---- online softmax over the 32 tokens; this thread holds 8 of them for rows gq and gq + 8
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < 4; ++n) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const bool ok = n * 8 + 2 * tq + j < n_tok;
        s[n][j] = ok ? s[n][j] * scale : -INFINITY;
        s[n][2 + j] = ok ? s[n][2 + j] * scale : -INFINITY;
        mx0 = fmaxf(mx0, s[n][j]);
        mx1 = fmaxf(mx1, s[n][2 + j]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);          // finite: token 0 of the pass is always valid
    const float al0 = (m0 == -INFINITY) ? 0.f : __expf(m0 - mn0);
    const float al1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - mn1);
    float sum0 = 0.f, sum1 = 0.f;
    uint32_t pfr[2][4];                                              // P as the A operand of the two 16-token k-steps
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const float p0 = __expf(s[n][0] - mn0), p1 = __expf(s[n][1] - mn0);
      const float p2 = __expf(s[n][2] - mn1), p3 = __expf(s[n][3] - mn1);
      sum0 += p0 + p1;
      sum1 += p2 + p3;
      pfr[n >> 1][(n & 1) * 2 + 0] = pa_pack_bf16(p0, p1);          // rows gq
      pfr[n >> 1][(n & 1) * 2 + 1] = pa_pack_bf16(p2, p3);          // rows gq + 8
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l0 = l0 * al0 + sum0;
    l1 = l1 * al1 + sum1;
    m0 = mn0;
    m1 = mn1;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      acc[n][0] *= al0; acc[n][1] *= al0; acc[n][2] *= al1; acc[n][3] *= al1;
    }
    // ---- O[16, D] += P[16, 32] V[32, D]
    if (more) pa_cp_wait<1>(); else pa_cp_wait<0>();                 // this pass's V tile has landed
    __syncwarp();
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {
        uint32_t bfr[4];
        // transposed 8x8 blocks: (tokens 16ks..+7, dims 16n2), (tokens +8, same dims), (tokens.., dims + 8), (+8, + 8)
        pa_ldsm_x4_t(vt_u32 + ((ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * KROW + n2 * 16 + (lane >> 4) * 8) * 2, bfr);
        pa_mma(acc[2 * n2], pfr[ks], bfr[0], bfr[1]);
        pa_mma(acc[2 * n2 + 1], pfr[ks], bfr[2], bfr[3]);
      }
    }
    __syncwarp();                                                    // every lane has read its V fragments
    if (more) request(v_cache, vt_u32);
  }

  // ---- merge the warps, write this slice's (max, sum, accumulator) per head
  __syncthreads();                            // every warp is done with its tile: the buffer becomes the merge area
  float (*acc_sh)[kMaxGroup][D] = reinterpret_cast<float (*)[kMaxGroup][D]>(big);
  if (tq == 0) {
    m_sh[warp][gq] = m0; l_sh[warp][gq] = l0;
    m_sh[warp][gq + 8] = m1; l_sh[warp][gq + 8] = l1;
  }
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    *reinterpret_cast<float2*>(&acc_sh[warp][gq][n * 8 + 2 * tq]) = make_float2(acc[n][0], acc[n][1]);
    *reinterpret_cast<float2*>(&acc_sh[warp][gq + 8][n * 8 + 2 * tq]) = make_float2(acc[n][2], acc[n][3]);
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
      num_slots RB_BOUNDS_ARG);
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
      max_blocks <= 0 || !scratch || num_blocks * block_size >= (1ll << 31))
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
  // dynamic shared memory: per warp a K and a V tile of 32 padded rows, plus the 16 padded query rows
  const int krow = head_dim + 8;
  const int smem = (rb::kPaWarps * 2 * 32 + rb::kMaxGroup) * krow * 2;
  static bool attr_set[64][2] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -3;
  if (!attr_set[dev][head_dim == 128]) {
    const cudaError_t e = head_dim == 128
        ? cudaFuncSetAttribute(rb::paged_decode_split_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
        : cudaFuncSetAttribute(rb::paged_decode_split_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev][head_dim == 128] = true;
  }
  for (int g0 = 0; g0 < group; g0 += rb::kMaxGroup) {     // groups wider than 16 heads take several passes
    const int gc = group - g0 < rb::kMaxGroup ? group - g0 : rb::kMaxGroup;
    if (head_dim == 128)
      rb::paged_decode_split_kernel<128><<<grid, rb::kPaWarps * 32, smem, stream>>>(Q, ld_q, K, V, block_tables, max_blocks,
                                                                                context_lens, heads, kv_heads, block_size,
                                                                                num_blocks, scale, g0, gc, scratch, nsplit RB_BOUNDS_ARG);
    else
      rb::paged_decode_split_kernel<64><<<grid, rb::kPaWarps * 32, smem, stream>>>(Q, ld_q, K, V, block_tables, max_blocks,
                                                                               context_lens, heads, kv_heads, block_size,
                                                                               num_blocks, scale, g0, gc, scratch, nsplit RB_BOUNDS_ARG);
  }
  dim3 mgrid(batch, heads);
  if (head_dim == 128)
    rb::paged_decode_merge_kernel<128><<<mgrid, 128, 0, stream>>>(scratch, context_lens, heads, nsplit, O, ld_o);
  else
    rb::paged_decode_merge_kernel<64><<<mgrid, 64, 0, stream>>>(scratch, context_lens, heads, nsplit, O, ld_o);
  return static_cast<int>(cudaGetLastError());
}
