// Expert-parallel token dispatch and combine over NVLink peer memory.
//
// The reference routes tokens on one device with host loops (crates/nn/src/moe.rs:277-370) and has no expert-parallel
// transport (crates/nn/src/moe.rs:478-520 only maps experts to ranks).  Here every rank writes its routed token rows
// directly into the receive buffer of the rank that owns the expert, at the row the grouped GEMM will read it from,
// and later pulls the expert outputs back and applies the routing weights, all with ordinary peer loads and stores.
#include "ep.h"

#include "rb_common.cuh"

namespace rb {

// one warp per (token, choice) pair; lanes cover the row with 16-byte vectors
__global__ void __launch_bounds__(256)
ep_push_rows_kernel(const __nv_bfloat16* __restrict__ src, int pairs, int k, int d, const int* __restrict__ dest_rank,
                    const int* __restrict__ dest_row, const float* __restrict__ scale, void* const* __restrict__ peer_bufs,
                    void* const* __restrict__ peer_counts) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n8 = d / 8;
  for (int p = blockIdx.x * warps_per_block + (threadIdx.x >> 5); p < pairs; p += gridDim.x * warps_per_block) {
    const int r = __ldg(dest_rank + p), row = __ldg(dest_row + p);
    if (r < 0 || row < 0) continue;
    const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<long long>(p / k) * d);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(peer_bufs[r]) + static_cast<long long>(row) * d);
    const float sc = scale ? __ldg(scale + p) : 1.f;
    for (int i = lane; i < n8; i += 32) {
      uint4 v = __ldg(s + i);
      if (scale) {
        uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          u[j] = pack_bf16x2(f.x * sc, f.y * sc);
        }
      }
      dst[i] = v;
    }
    if (peer_counts != nullptr) {
      // the row is complete: count it for the 128-row tile it belongs to, so that the owner's grouped GEMM can start on
      // that tile as soon as all of its rows have arrived
      __syncwarp();
      if (lane == 0) {
        __threadfence_system();
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(reinterpret_cast<unsigned int*>(peer_counts[r]) + (row >> 7)), "r"(1u) : "memory");
      }
    }
  }
}

// one warp per token: pulls its k expert rows (peer loads) and folds them in choice order
__global__ void __launch_bounds__(256)
ep_pull_combine_kernel(__nv_bfloat16* __restrict__ out, int tokens, int k, int d, const int* __restrict__ dest_rank,
                       const int* __restrict__ dest_row, const float* __restrict__ w,
                       const __nv_bfloat16* __restrict__ residual, void* const* __restrict__ peer_bufs) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n8 = d / 8;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < tokens; t += gridDim.x * warps_per_block) {
    for (int i = lane; i < n8; i += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (residual) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(residual + static_cast<long long>(t) * d) + i);
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(u[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
      }
      for (int c = 0; c < k; ++c) {
        const int p = t * k + c;
        const int r = __ldg(dest_rank + p), row = __ldg(dest_row + p);
        if (r < 0 || row < 0) continue;
        const float wc = w ? __ldg(w + p) : 1.f;
        const uint4 v = *(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(peer_bufs[r]) +
                                                          static_cast<long long>(row) * d) + i);
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          acc[2 * j] = fmaf(wc, f.x, acc[2 * j]);
          acc[2 * j + 1] = fmaf(wc, f.y, acc[2 * j + 1]);
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out + static_cast<long long>(t) * d)[i] = o;
    }
  }
}

// one warp per (token, choice) pair
__global__ void __launch_bounds__(256)
ep_pull_dot_kernel(float* __restrict__ dw, const __nv_bfloat16* __restrict__ dy, int pairs, int k, int d,
                   const int* __restrict__ dest_rank, const int* __restrict__ dest_row, void* const* __restrict__ peer_bufs) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n8 = d / 8;
  for (int p = blockIdx.x * warps_per_block + (threadIdx.x >> 5); p < pairs; p += gridDim.x * warps_per_block) {
    const int r = __ldg(dest_rank + p), row = __ldg(dest_row + p);
    float acc = 0.f;
    if (r >= 0 && row >= 0) {
      const uint4* a = reinterpret_cast<const uint4*>(dy + static_cast<long long>(p / k) * d);
      const uint4* b = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(peer_bufs[r]) +
                                                      static_cast<long long>(row) * d);
      for (int i = lane; i < n8; i += 32) {
        const uint4 x = __ldg(a + i);
        const uint4 y = b[i];
        const uint32_t* ux = reinterpret_cast<const uint32_t*>(&x);
        const uint32_t* uy = reinterpret_cast<const uint32_t*>(&y);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fx = unpack_bf16x2(ux[j]), fy = unpack_bf16x2(uy[j]);
          acc = fmaf(fx.x, fy.x, acc);
          acc = fmaf(fx.y, fy.y, acc);
        }
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) dw[p] = acc;
  }
}

__global__ void __launch_bounds__(256)
ep_zero_padding_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ offsets, const int* __restrict__ counts,
                       int d) {
  const int e = blockIdx.x;
  const int first = __ldg(offsets + e) + __ldg(counts + e), last = __ldg(offsets + e + 1);
  const long long n8 = static_cast<long long>(last - first) * d / 8;
  uint4* p = reinterpret_cast<uint4*>(buf + static_cast<long long>(first) * d);
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  for (long long i = threadIdx.x; i < n8; i += blockDim.x) p[i] = z;
}

}  // namespace rb

namespace {
int grid_for(long long warps_needed) {
  long long blocks = (warps_needed + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}
bool bad_row(const void* p, int d) { return !p || (reinterpret_cast<uintptr_t>(p) & 15) || d <= 0 || (d % 8); }
}  // namespace

RB_API int rb_ep_push_rows(const void* src, int tokens, int k, int d, const int* dest_rank, const int* dest_row,
                           const float* scale, void* const* peer_bufs_dev, void* const* peer_counts_dev, void* stream_v) {
  if (bad_row(src, d) || tokens < 0 || k <= 0 || !dest_rank || !dest_row || !peer_bufs_dev) return -1;
  if (tokens == 0) return 0;
  const int pairs = tokens * k;
  rb::ep_push_rows_kernel<<<grid_for(pairs), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), pairs, k, d, dest_rank, dest_row, scale, peer_bufs_dev, peer_counts_dev);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_ep_pull_combine(void* out, int tokens, int k, int d, const int* dest_rank, const int* dest_row, const float* w,
                              const void* residual, void* const* peer_bufs_dev, void* stream_v) {
  if (bad_row(out, d) || tokens < 0 || k <= 0 || !dest_rank || !dest_row || !peer_bufs_dev) return -1;
  if (residual && (reinterpret_cast<uintptr_t>(residual) & 15)) return -1;
  if (tokens == 0) return 0;
  rb::ep_pull_combine_kernel<<<grid_for(tokens), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<__nv_bfloat16*>(out), tokens, k, d, dest_rank, dest_row, w,
      reinterpret_cast<const __nv_bfloat16*>(residual), peer_bufs_dev);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_ep_pull_dot(float* dw, const void* dy, int tokens, int k, int d, const int* dest_rank, const int* dest_row,
                          void* const* peer_bufs_dev, void* stream_v) {
  if (bad_row(dy, d) || !dw || tokens < 0 || k <= 0 || !dest_rank || !dest_row || !peer_bufs_dev) return -1;
  if (tokens == 0) return 0;
  const int pairs = tokens * k;
  rb::ep_pull_dot_kernel<<<grid_for(pairs), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      dw, reinterpret_cast<const __nv_bfloat16*>(dy), pairs, k, d, dest_rank, dest_row, peer_bufs_dev);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_ep_zero_padding(void* buf, const int* offsets, const int* counts, int num_local_experts, int d,
                              void* stream_v) {
  if (bad_row(buf, d) || !offsets || !counts || num_local_experts <= 0) return -1;
  rb::ep_zero_padding_kernel<<<num_local_experts, 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<__nv_bfloat16*>(buf), offsets, counts, d);
  return static_cast<int>(cudaGetLastError());
}
