// Token (+ learned position) embedding: row gather forward, deterministic scatter-add backward.
//
// The backward pass never uses floating-point atomics.  Token positions are bucketed by id with a
// counting sort (integer atomics only), each bucket is then visited in ascending token order by one
// warp, so the fp32 sum into a table row has a fixed order.  Replaces gather_rows / the host-side
// scatter-add of the reference (crates/autodiff/src/lib.rs:847-930; shaders.wgsl:924-996).
#include "embedding.h"

#include <limits.h>

#include "rb_common.cuh"

namespace rb {

__global__ void __launch_bounds__(128)
embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ wte,
                     const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out, long long tokens, int dim,
                     int seq_len, long long vocab RB_BOUNDS_PARAM) {
  const int chunks = dim / 8;
  const long long total = tokens * chunks;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long t = i / chunks;
    const int c = static_cast<int>(i - t * chunks) * 8;
    long long id = ids[t];
    if (id < 0 || id >= vocab) {         // out-of-range ids read row 0 instead of faulting
      if (c == 0) RB_BOUNDS_HIT(101);
      id = 0;
    }
    uint4 a = __ldg(reinterpret_cast<const uint4*>(wte + id * dim + c));
    if (wpe) {
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(wpe + (t % seq_len) * dim + c));
      float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
      float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
      a.x = pack_bf16x2(a0.x + b0.x, a0.y + b0.y); a.y = pack_bf16x2(a1.x + b1.x, a1.y + b1.y);
      a.z = pack_bf16x2(a2.x + b2.x, a2.y + b2.y); a.w = pack_bf16x2(a3.x + b3.x, a3.y + b3.y);
    }
    *reinterpret_cast<uint4*>(out + t * dim + c) = a;
  }
}

__global__ void hist_kernel(const long long* __restrict__ ids, long long tokens, long long vocab, int* counts) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < tokens; t += stride) {
    const long long id = ids[t];
    if (id >= 0 && id < vocab) atomicAdd(&counts[id], 1);
  }
}

// single CTA exclusive scan; offsets[vocab] = total
__global__ void __launch_bounds__(1024) scan_kernel(const int* __restrict__ counts, int* __restrict__ offsets, long long vocab) {
  __shared__ int sh[1024];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (long long base = 0; base < vocab; base += 1024) {
    const long long i = base + threadIdx.x;
    const int v = i < vocab ? counts[i] : 0;
    sh[threadIdx.x] = v;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
      const int t = threadIdx.x >= o ? sh[threadIdx.x - o] : 0;
      __syncthreads();
      sh[threadIdx.x] += t;
      __syncthreads();
    }
    if (i < vocab) offsets[i] = carry + sh[threadIdx.x] - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry += sh[1023];
    __syncthreads();
  }
  if (threadIdx.x == 0) offsets[vocab] = carry;
}

__global__ void fill_kernel(const long long* __restrict__ ids, long long tokens, long long vocab,
                            const int* __restrict__ offsets, int* cursor, int* __restrict__ perm) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < tokens; t += stride) {
    const long long id = ids[t];
    if (id >= 0 && id < vocab) {
      const int pos = offsets[id] + atomicAdd(&cursor[id], 1);
      perm[pos] = static_cast<int>(t);
    }
  }
}

// One warp per table row: order the bucket by token index, then sum dy rows in that order.
__global__ void __launch_bounds__(128)
scatter_rows_kernel(const __nv_bfloat16* __restrict__ dy, const int* __restrict__ offsets, const int* __restrict__ perm,
                    int* __restrict__ sorted, float* __restrict__ dw, int dim, long long vocab) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= vocab) return;
  const int lo = offsets[row], hi = offsets[row + 1];
  const int count = hi - lo;
  if (count == 0) return;
  int last = -1;
  for (int j = 0; j < count; ++j) {   // selection by repeated minimum: O(count^2 / 32), buckets are short
    int cand = INT_MAX;
    for (int k = lane; k < count; k += 32) {
      const int x = perm[lo + k];
      if (x > last && x < cand) cand = x;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    if (lane == 0) sorted[lo + j] = cand;
    last = cand;
  }
  __syncwarp();
  const int chunks = dim / 8;
  for (int c = lane; c < chunks; c += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < count; ++j) {
      const long long t = sorted[lo + j];
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(dy + t * dim + c * 8));
      float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
      acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
      acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
    }
    float* w = dw + row * dim + c * 8;
    float4 w0 = *reinterpret_cast<float4*>(w), w1 = *reinterpret_cast<float4*>(w + 4);
    w0.x += acc[0]; w0.y += acc[1]; w0.z += acc[2]; w0.w += acc[3];
    w1.x += acc[4]; w1.y += acc[5]; w1.z += acc[6]; w1.w += acc[7];
    *reinterpret_cast<float4*>(w) = w0;
    *reinterpret_cast<float4*>(w + 4) = w1;
  }
}

// dwpe[s, c] += sum_b dy[b*seq_len + s, c]
__global__ void __launch_bounds__(128)
pos_grad_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ dwpe, long long tokens, int dim, int seq_len) {
  const int chunks = dim / 8;
  const long long total = static_cast<long long>(seq_len) * chunks;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long s = i / chunks;
  const int c = static_cast<int>(i - s * chunks) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (long long t = s; t < tokens; t += seq_len) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(dy + t * dim + c));
    float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
    acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
    acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
  }
  float* w = dwpe + s * dim + c;
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j] += acc[j];
}

}  // namespace rb

RB_API int rb_embedding_fwd(const long long* ids, const void* wte, const void* wpe, void* out, long long tokens,
                            int dim, int seq_len, long long vocab, void* stream_v) {
  if (tokens <= 0 || dim <= 0 || (dim & 7) || vocab <= 0 || (wpe && seq_len <= 0)) return -1;
  if ((reinterpret_cast<uintptr_t>(wte) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(wpe)) & 15) return -2;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const long long total = tokens * (dim / 8);
  long long blocks = (total + 127) / 128;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  rb::embedding_fwd_kernel<<<static_cast<int>(blocks), 128, 0, stream>>>(
      ids, reinterpret_cast<const __nv_bfloat16*>(wte), reinterpret_cast<const __nv_bfloat16*>(wpe),
      reinterpret_cast<__nv_bfloat16*>(out), tokens, dim, seq_len < 1 ? 1 : seq_len, vocab RB_BOUNDS_ARG);
  return static_cast<int>(cudaGetLastError());
}

RB_API long long rb_embedding_bwd_scratch_ints(long long tokens, long long vocab) {
  // counts[vocab] | cursor[vocab] | offsets[vocab + 1] | perm[tokens] | sorted[tokens]
  return 3 * vocab + 1 + 2 * tokens;
}

RB_API int rb_embedding_bwd(const long long* ids, const void* dy, float* dwte, float* dwpe, int* scratch,
                            long long tokens, int dim, int seq_len, long long vocab, void* stream_v) {
  if (tokens <= 0 || dim <= 0 || (dim & 7) || vocab <= 0 || !scratch || tokens > INT_MAX) return -1;
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dwte) | reinterpret_cast<uintptr_t>(dwpe)) & 15) return -2;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  int* counts = scratch;
  int* cursor = counts + vocab;
  int* offsets = cursor + vocab;
  int* perm = offsets + vocab + 1;
  int* sorted = perm + tokens;
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * 2 * vocab, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  int tb = static_cast<int>((tokens + 255) / 256);
  if (tb > 148 * 8) tb = 148 * 8;
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  if (dwte) {
    rb::hist_kernel<<<tb, 256, 0, stream>>>(ids, tokens, vocab, counts);
    rb::scan_kernel<<<1, 1024, 0, stream>>>(counts, offsets, vocab);
    rb::fill_kernel<<<tb, 256, 0, stream>>>(ids, tokens, vocab, offsets, cursor, perm);
    rb::scatter_rows_kernel<<<static_cast<int>((vocab + 3) / 4), 128, 0, stream>>>(DY, offsets, perm, sorted, dwte, dim, vocab);
  }
  if (dwpe) {
    const long long total = static_cast<long long>(seq_len) * (dim / 8);
    rb::pos_grad_kernel<<<static_cast<int>((total + 127) / 128), 128, 0, stream>>>(DY, dwpe, tokens, dim, seq_len);
  }
  return static_cast<int>(cudaGetLastError());
}
