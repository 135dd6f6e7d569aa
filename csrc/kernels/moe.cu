// Mixture-of-experts routing: router softmax + top-k, a deterministic token -> expert permutation plan whose
// expert segments are padded to whole GEMM tiles, gather / combine with the routing weights, and the backward
// passes of all of them.  The grouped expert GEMM itself is the tcgen05 kernel run over the permuted buffer
// (gemm_tcgen05.cu, grouped mode).
//
// The reference's gating picks experts as `i % E` and dispatches every token to every expert
// (crates/nn/src/moe.rs:122-141,344-348); expert-choice and shared-expert routing run on the host
// (crates/nn/src/expert_choice.rs:205-315, crates/nn/src/shared_expert.rs:279-375).
#include "moe.h"

#include <float.h>

#include "rb_common.cuh"

namespace rb {

constexpr int kMaxK = 8;

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int T, int E, int k, int renorm, int* __restrict__ idx,
                 float* __restrict__ w, float* __restrict__ probs_out) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const float* x = logits + static_cast<long long>(t) * E;
  float v0 = lane < E ? x[lane] : -INFINITY;
  float v1 = lane + 32 < E ? x[lane + 32] : -INFINITY;
  const float mx = warp_max(fmaxf(v0, v1));
  float p0 = lane < E ? __expf(v0 - mx) : 0.f;
  float p1 = lane + 32 < E ? __expf(v1 - mx) : 0.f;
  const float inv = 1.f / warp_sum(p0 + p1);
  p0 *= inv;
  p1 *= inv;
  if (probs_out) {
    if (lane < E) probs_out[static_cast<long long>(t) * E + lane] = p0;
    if (lane + 32 < E) probs_out[static_cast<long long>(t) * E + lane + 32] = p1;
  }
  float sel_p[kMaxK];
  int sel_i[kMaxK];
  float tot = 0.f;
  float c0 = lane < E ? p0 : -1.f, c1 = lane + 32 < E ? p1 : -1.f;
  for (int j = 0; j < k; ++j) {
    // warp arg-max with ties to the lower expert index
    float bv = c0;
    int bi = lane;
    if (c1 > bv) { bv = c1; bi = lane + 32; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    sel_p[j] = bv;
    sel_i[j] = bi;
    tot += bv;
    if (bi == lane) c0 = -1.f;
    if (bi == lane + 32) c1 = -1.f;
  }
  if (lane == 0) {
    for (int j = 0; j < k; ++j) {
      idx[static_cast<long long>(t) * k + j] = sel_i[j];
      w[static_cast<long long>(t) * k + j] = renorm ? sel_p[j] / tot : sel_p[j];
    }
  }
}

__global__ void __launch_bounds__(128)
moe_route_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ idx, const float* __restrict__ w,
                     const float* __restrict__ dw, const int* __restrict__ counts, int T, int E, int k, int renorm,
                     float aux_grad_scale, float* __restrict__ dlogits) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const float* p = probs + static_cast<long long>(t) * E;
  float dp[2] = {0.f, 0.f};
  // gradient through the (renormalised) selected weights
  float S = 0.f, dot = 0.f;
  for (int j = 0; j < k; ++j) {
    const int e = idx[static_cast<long long>(t) * k + j];
    S += p[e];
    dot += dw[static_cast<long long>(t) * k + j] * w[static_cast<long long>(t) * k + j];
  }
  for (int j = 0; j < k; ++j) {
    const int e = idx[static_cast<long long>(t) * k + j];
    const float g = dw[static_cast<long long>(t) * k + j];
    const float d = renorm ? (g - dot) / S : g;
    if (e == lane) dp[0] += d;
    if (e == lane + 32) dp[1] += d;
  }
  // load-balancing loss: d aux / d p[t, e] = E * f_e / T
  const float denom = static_cast<float>(T) * static_cast<float>(k);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int e = lane + 32 * h;
    if (e < E) dp[h] += aux_grad_scale * static_cast<float>(E) * (static_cast<float>(counts[e]) / denom) / static_cast<float>(T);
  }
  // softmax backward
  const float pv0 = lane < E ? p[lane] : 0.f, pv1 = lane + 32 < E ? p[lane + 32] : 0.f;
  const float s = warp_sum(dp[0] * pv0 + dp[1] * pv1);
  if (lane < E) dlogits[static_cast<long long>(t) * E + lane] = pv0 * (dp[0] - s);
  if (lane + 32 < E) dlogits[static_cast<long long>(t) * E + lane + 32] = pv1 * (dp[1] - s);
}

// ---- permutation plan ---------------------------------------------------------------------------------------
__device__ __forceinline__ int block_scan_excl(int v, int* sh, int& total) {
  // exclusive scan over 1024 threads; sh has 1024 ints
  sh[threadIdx.x] = v;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const int t = threadIdx.x >= o ? sh[threadIdx.x - o] : 0;
    __syncthreads();
    sh[threadIdx.x] += t;
    __syncthreads();
  }
  const int incl = sh[threadIdx.x];
  total = sh[1023];
  __syncthreads();
  return incl - v;
}

__global__ void __launch_bounds__(1024) moe_count_kernel(const int* __restrict__ idx, int slots, int* __restrict__ counts) {
  __shared__ int sh[32];
  const int e = blockIdx.x;
  int c = 0;
  for (int s = threadIdx.x; s < slots; s += 1024) c += (idx[s] == e);
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int i = 0; i < 32; ++i) t += sh[i];
    counts[e] = t;
  }
}

__global__ void moe_offsets_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                                   int* __restrict__ tile_expert, int* __restrict__ num_tiles, int max_tiles) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int off = 0, tile = 0;
  for (int e = 0; e < E; ++e) {
    offsets[e] = off;
    const int padded = (counts[e] + RB_MOE_ROW_ALIGN - 1) / RB_MOE_ROW_ALIGN * RB_MOE_ROW_ALIGN;
    for (int i = 0; i < padded / 128 && tile < max_tiles; ++i) tile_expert[tile++] = e;
    off += padded;
  }
  offsets[E] = off;
  num_tiles[0] = tile;
  for (int i = tile; i < max_tiles; ++i) tile_expert[i] = -1;
}

__global__ void __launch_bounds__(1024)
moe_assign_kernel(const int* __restrict__ idx, int slots, const int* __restrict__ offsets, int* __restrict__ slot_pos,
                  int* __restrict__ row_slot) {
  __shared__ int sh[1024];
  const int e = blockIdx.x;
  int base = offsets[e];
  for (int s0 = 0; s0 < slots; s0 += 1024) {
    const int s = s0 + threadIdx.x;
    const int match = (s < slots && idx[s] == e) ? 1 : 0;
    int total;
    const int rank = block_scan_excl(match, sh, total);
    if (match) {
      slot_pos[s] = base + rank;
      row_slot[base + rank] = s;
    }
    base += total;
  }
}

__global__ void __launch_bounds__(128)
moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_slot, const float* __restrict__ slot_scale,
                  __nv_bfloat16* __restrict__ xp, int max_rows, int k, int dim, const int* __restrict__ total_rows) {
  const int chunks = dim / 8;
  const int rows = min(max_rows, total_rows[0]);
  const long long total = static_cast<long long>(rows) * chunks;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int r = static_cast<int>(i / chunks);
    const int c = static_cast<int>(i - static_cast<long long>(r) * chunks) * 8;
    const int s = row_slot[r];
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (s >= 0) {
      v = *reinterpret_cast<const uint4*>(x + static_cast<long long>(s / k) * dim + c);
      if (slot_scale) {
        const float sc = slot_scale[s];
        uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(pv[j]);
          pv[j] = pack_bf16x2(f.x * sc, f.y * sc);
        }
      }
    }
    *reinterpret_cast<uint4*>(xp + static_cast<long long>(r) * dim + c) = v;
  }
}

__global__ void __launch_bounds__(128)
moe_combine_kernel(const __nv_bfloat16* __restrict__ yp, const int* __restrict__ slot_pos, const float* __restrict__ w,
                   const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ y, int T, int k, int dim) {
  const int chunks = dim / 8;
  const long long total = static_cast<long long>(T) * chunks;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int t = static_cast<int>(i / chunks);
    const int c = static_cast<int>(i - static_cast<long long>(t) * chunks) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (residual) {
      const uint4 u = *reinterpret_cast<const uint4*>(residual + static_cast<long long>(t) * dim + c);
      const uint32_t* pu = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(pu[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
    }
    for (int j = 0; j < k; ++j) {     // fixed order: reproducible
      const int s = t * k + j;
      const float wj = w ? w[s] : 1.f;
      const uint4 u = *reinterpret_cast<const uint4*>(yp + static_cast<long long>(slot_pos[s]) * dim + c);
      const uint32_t* pu = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
      for (int q = 0; q < 4; ++q) { const float2 f = unpack_bf16x2(pu[q]); acc[2 * q] += wj * f.x; acc[2 * q + 1] += wj * f.y; }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(y + static_cast<long long>(t) * dim + c) = o;
  }
}

__global__ void __launch_bounds__(128)
moe_weight_grad_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ yp, const int* __restrict__ slot_pos,
                       float* __restrict__ dw, int slots, int k, int dim) {
  const int lane = threadIdx.x & 31;
  const int s = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (s >= slots) return;
  const __nv_bfloat16* a = dy + static_cast<long long>(s / k) * dim;
  const __nv_bfloat16* b = yp + static_cast<long long>(slot_pos[s]) * dim;
  float acc = 0.f;
  for (int c = lane * 8; c < dim; c += 256) {
    const uint4 ua = *reinterpret_cast<const uint4*>(a + c), ub = *reinterpret_cast<const uint4*>(b + c);
    const uint32_t* pa = reinterpret_cast<const uint32_t*>(&ua);
    const uint32_t* pb = reinterpret_cast<const uint32_t*>(&ub);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = unpack_bf16x2(pa[j]), fb = unpack_bf16x2(pb[j]);
      acc += fa.x * fb.x + fa.y * fb.y;
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) dw[s] = acc;
}

inline int grid1d(long long n, int per_block) {
  long long b = (n + per_block - 1) / per_block;
  if (b > 148LL * 32) b = 148LL * 32;
  return static_cast<int>(b < 1 ? 1 : b);
}

}  // namespace rb

#define RB_ST reinterpret_cast<cudaStream_t>(stream_v)

RB_API int rb_moe_route(const float* logits, int T, int E, int k, int renorm, int* idx, float* w, float* probs_out, void* stream_v) {
  if (T <= 0 || E <= 0 || E > 64 || k <= 0 || k > rb::kMaxK || k > E) return -1;
  rb::moe_route_kernel<<<(T + 3) / 4, 128, 0, RB_ST>>>(logits, T, E, k, renorm, idx, w, probs_out);
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_moe_route_bwd(const float* probs, const int* idx, const float* w, const float* dw, const int* counts, int T,
                            int E, int k, int renorm, float aux_grad_scale, float* dlogits, void* stream_v) {
  if (T <= 0 || E <= 0 || E > 64 || k <= 0 || k > rb::kMaxK) return -1;
  rb::moe_route_bwd_kernel<<<(T + 3) / 4, 128, 0, RB_ST>>>(probs, idx, w, dw, counts, T, E, k, renorm, aux_grad_scale, dlogits);
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_moe_plan(const int* idx, int T, int E, int k, int* counts, int* offsets, int* slot_pos, int* row_slot,
                       int* tile_expert, int* num_tiles, int max_rows, void* stream_v) {
  if (T <= 0 || E <= 0 || k <= 0 || max_rows < T * k + E * RB_MOE_ROW_ALIGN || (max_rows % 128)) return -1;
  cudaError_t e = cudaMemsetAsync(row_slot, 0xFF, sizeof(int) * static_cast<size_t>(max_rows), RB_ST);
  if (e != cudaSuccess) return static_cast<int>(e);
  rb::moe_count_kernel<<<E, 1024, 0, RB_ST>>>(idx, T * k, counts);
  rb::moe_offsets_kernel<<<1, 32, 0, RB_ST>>>(counts, E, offsets, tile_expert, num_tiles, max_rows / 128);
  rb::moe_assign_kernel<<<E, 1024, 0, RB_ST>>>(idx, T * k, offsets, slot_pos, row_slot);
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_moe_gather(const void* x, const int* row_slot, const float* slot_scale, void* xp, int max_rows, int k, int dim,
                         const int* offsets_last, void* stream_v) {
  if (max_rows <= 0 || dim <= 0 || (dim % 8) || !offsets_last) return -1;
  rb::moe_gather_kernel<<<rb::grid1d(static_cast<long long>(max_rows) * (dim / 8), 128), 128, 0, RB_ST>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), row_slot, slot_scale, reinterpret_cast<__nv_bfloat16*>(xp), max_rows, k, dim,
      offsets_last);
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_moe_combine(const void* yp, const int* slot_pos, const float* w, const void* residual, void* y, int T, int k,
                          int dim, void* stream_v) {
  if (T <= 0 || dim <= 0 || (dim % 8)) return -1;
  rb::moe_combine_kernel<<<rb::grid1d(static_cast<long long>(T) * (dim / 8), 128), 128, 0, RB_ST>>>(
      reinterpret_cast<const __nv_bfloat16*>(yp), slot_pos, w, reinterpret_cast<const __nv_bfloat16*>(residual),
      reinterpret_cast<__nv_bfloat16*>(y), T, k, dim);
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_moe_weight_grad(const void* dy, const void* yp, const int* slot_pos, float* dw, int T, int k, int dim, void* stream_v) {
  if (T <= 0 || dim <= 0 || (dim % 8)) return -1;
  rb::moe_weight_grad_kernel<<<(T * k + 3) / 4, 128, 0, RB_ST>>>(reinterpret_cast<const __nv_bfloat16*>(dy),
                                                                  reinterpret_cast<const __nv_bfloat16*>(yp), slot_pos, dw,
                                                                  T * k, k, dim);
  return static_cast<int>(cudaGetLastError());
}
