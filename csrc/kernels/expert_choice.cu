// Expert-choice routing (crates/nn/src/expert_choice.rs:205-238: every expert takes its `capacity` highest-affinity
// tokens).  Kernels:
//   rb_ec_select       per expert, the `cap` tokens with the largest probability, by a radix select over the float bits
//                      (four 8-bit passes, one CTA per expert); ties at the threshold go to the lower token index; the
//                      chosen tokens come out in ascending token order with their probabilities
//   rb_ec_table        table[t, e] = position of token t in expert e's list, or -1
//   rb_ec_combine      out[t, :] = sum over e (ascending) of gate[e, s] * y[e * cap + s, :] with s = table[t, e]: a gather per
//                      token in a fixed order, no atomics (gate == NULL: unit weights, which is also the backward of the
//                      row gather that feeds the experts)
//   rb_ec_combine_bwd  dy[j, :] = gate[j] * dout[idx[j], :] and dgate[j] = <dout[idx[j], :], y[j, :]>, one warp per row
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "expert_choice.h"
#include "rb_common.cuh"

namespace rb {

__device__ __forceinline__ uint32_t ec_key(float p) {
  // order-preserving map of a float to an unsigned integer (probabilities are >= 0, NaN sorts last as 0)
  if (!(p == p)) return 0u;
  uint32_t u = __float_as_uint(p);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// probs [T, E] fp32 (row per token).  One CTA of 1024 threads per expert.
__global__ void __launch_bounds__(1024)
ec_select_kernel(const float* __restrict__ probs, int T, int E, int cap, long long* __restrict__ idx, float* __restrict__ gate) {
  __shared__ unsigned int hist[256];
  __shared__ unsigned int s_prefix, s_need, s_count;
  __shared__ unsigned int warp_tot[32];
  const int e = blockIdx.x;
  const int tid = threadIdx.x;
  // ---- radix select of the cap-th largest key
  uint32_t prefix = 0, mask = 0;
  unsigned int need = static_cast<unsigned int>(cap);
  for (int pass = 3; pass >= 0; --pass) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const int shift = pass * 8;
    for (int t = tid; t < T; t += blockDim.x) {
      const uint32_t k = ec_key(probs[static_cast<long long>(t) * E + e]);
      if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 0xff], 1u);          // integer counts: order-independent
    }
    __syncthreads();
    if (tid == 0) {
      unsigned int acc = 0;
      int b = 255;
      for (; b > 0; --b) {
        if (acc + hist[b] >= need) break;
        acc += hist[b];
      }
      s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      s_need = need - acc;
    }
    __syncthreads();
    prefix = s_prefix;
    need = s_need;
    mask |= 0xffu << shift;
    __syncthreads();
  }
  // prefix is now the key of the cap-th largest element; `need` of the elements equal to it are taken (lowest indices)
  const uint32_t thr = prefix;
  // ---- ordered compaction: chunks of blockDim tokens, prefix sums inside the CTA
  if (tid == 0) s_count = 0;
  __shared__ unsigned int s_eq_taken;
  if (tid == 0) s_eq_taken = 0;
  __syncthreads();
  for (int base = 0; base < T; base += blockDim.x) {
    const int t = base + tid;
    float p = 0.f;
    uint32_t k = 0;
    if (t < T) { p = probs[static_cast<long long>(t) * E + e]; k = ec_key(p); }
    const bool gt = t < T && k > thr, eq = t < T && k == thr;
    // rank of this thread among the "equal" elements of the chunk, then among the taken elements
    const unsigned int lane = tid & 31, warp = tid >> 5;
    const unsigned int eq_ballot = __ballot_sync(0xffffffffu, eq);
    unsigned int eq_before = __popc(eq_ballot & ((1u << lane) - 1));
    if (lane == 0) warp_tot[warp] = __popc(eq_ballot);
    __syncthreads();
    unsigned int eq_base = s_eq_taken;
    for (unsigned int w = 0; w < warp; ++w) eq_base += warp_tot[w];
    unsigned int eq_chunk = 0;
    for (unsigned int w = 0; w < (blockDim.x >> 5); ++w) eq_chunk += warp_tot[w];
    const bool take = gt || (eq && eq_base + eq_before < need);
    __syncthreads();
    const unsigned int tk_ballot = __ballot_sync(0xffffffffu, take);
    const unsigned int tk_before = __popc(tk_ballot & ((1u << lane) - 1));
    if (lane == 0) warp_tot[warp] = __popc(tk_ballot);
    __syncthreads();
    unsigned int pos = s_count;
    for (unsigned int w = 0; w < warp; ++w) pos += warp_tot[w];
    unsigned int tk_chunk = 0;
    for (unsigned int w = 0; w < (blockDim.x >> 5); ++w) tk_chunk += warp_tot[w];
    if (take && pos + tk_before < static_cast<unsigned int>(cap)) {
      idx[static_cast<long long>(e) * cap + pos + tk_before] = t;
      gate[static_cast<long long>(e) * cap + pos + tk_before] = p;
    }
    __syncthreads();
    if (tid == 0) { s_count += tk_chunk; s_eq_taken += eq_chunk; }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256)
ec_table_kernel(const long long* __restrict__ idx, int n, int T, int E, int cap, int* __restrict__ table) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const long long t = idx[j];
  if (t < 0 || t >= T) return;
  table[t * E + j / cap] = j % cap;          // an expert's tokens are distinct: every entry has one writer
}

template <typename OutT>
__global__ void __launch_bounds__(256)
ec_combine_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ gate, const int* __restrict__ table,
                  OutT* __restrict__ out, int T, int E, int cap, int d) {
  const int d8 = d / 8;
  const long long total = static_cast<long long>(T) * d8;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const long long t = i / d8;
    const int c = static_cast<int>(i - t * d8) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int e = 0; e < E; ++e) {
      const int s = __ldg(table + t * E + e);
      if (s < 0) continue;
      const long long j = static_cast<long long>(e) * cap + s;
      const float g = gate ? __ldg(gate + j) : 1.f;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(y + j * d + c));
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), cc = unpack_bf16x2(v.z), dd = unpack_bf16x2(v.w);
      acc[0] += g * a.x; acc[1] += g * a.y; acc[2] += g * b.x; acc[3] += g * b.y;
      acc[4] += g * cc.x; acc[5] += g * cc.y; acc[6] += g * dd.x; acc[7] += g * dd.y;
    }
    if (sizeof(OutT) == 4) {
      float* op = reinterpret_cast<float*>(out) + t * d + c;
      reinterpret_cast<float4*>(op)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      reinterpret_cast<float4*>(op)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + t * d + c) = o;
    }
  }
}

// one warp per chosen row j
__global__ void __launch_bounds__(256)
ec_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const long long* __restrict__ idx, const float* __restrict__ gate,
                      const __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ dy, float* __restrict__ dgate, int n, int T,
                      int d) {
  const int j = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (j >= n) return;
  const long long t = idx[j];
  const bool ok = t >= 0 && t < T;
  const float g = gate ? gate[j] : 1.f;
  float dot = 0.f;
  for (int c = lane * 8; c < d; c += 256) {
    uint4 dv = make_uint4(0, 0, 0, 0);
    if (ok) dv = __ldg(reinterpret_cast<const uint4*>(dout + t * d + c));
    const float2 a = unpack_bf16x2(dv.x), b = unpack_bf16x2(dv.y), cc = unpack_bf16x2(dv.z), dd = unpack_bf16x2(dv.w);
    if (y != nullptr) {
      const uint4 yv = __ldg(reinterpret_cast<const uint4*>(y + static_cast<long long>(j) * d + c));
      const float2 ya = unpack_bf16x2(yv.x), yb = unpack_bf16x2(yv.y), yc = unpack_bf16x2(yv.z), yd = unpack_bf16x2(yv.w);
      dot += a.x * ya.x + a.y * ya.y + b.x * yb.x + b.y * yb.y + cc.x * yc.x + cc.y * yc.y + dd.x * yd.x + dd.y * yd.y;
    }
    uint4 o;
    o.x = pack_bf16x2(g * a.x, g * a.y); o.y = pack_bf16x2(g * b.x, g * b.y);
    o.z = pack_bf16x2(g * cc.x, g * cc.y); o.w = pack_bf16x2(g * dd.x, g * dd.y);
    *reinterpret_cast<uint4*>(dy + static_cast<long long>(j) * d + c) = o;
  }
  if (dgate != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) dgate[j] = dot;
  }
}

}  // namespace rb

RB_API int rb_ec_select(const float* probs, int T, int E, int cap, long long* idx, float* gate, void* stream) {
  if (!probs || !idx || !gate || T <= 0 || E <= 0 || cap <= 0 || cap > T) return -1;
  rb::ec_select_kernel<<<E, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(probs, T, E, cap, idx, gate);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_ec_table(const long long* idx, int T, int E, int cap, int* table, void* stream_v) {
  if (!idx || !table || T <= 0 || E <= 0 || cap <= 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  cudaError_t e = cudaMemsetAsync(table, 0xff, static_cast<size_t>(T) * E * sizeof(int), stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int n = E * cap;
  rb::ec_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(idx, n, T, E, cap, table);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_ec_combine(const void* y, const float* gate, const int* table, void* out, int T, int E, int cap, int d, int out_f32,
                         void* stream_v) {
  if (!y || !table || !out || T <= 0 || E <= 0 || cap <= 0 || d <= 0 || (d & 7)) return -1;
  if ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15) return -2;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const long long total = static_cast<long long>(T) * (d / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (out_f32)
    rb::ec_combine_kernel<float><<<static_cast<int>(blocks), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(y), gate, table,
                                                                                 reinterpret_cast<float*>(out), T, E, cap, d);
  else
    rb::ec_combine_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(y), gate, table, reinterpret_cast<__nv_bfloat16*>(out), T, E, cap, d);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_ec_combine_bwd(const void* dout, const long long* idx, const float* gate, const void* y, void* dy, float* dgate, int n,
                             int T, int d, void* stream) {
  if (!dout || !idx || !dy || n <= 0 || T <= 0 || d <= 0 || (d & 7)) return -1;
  if ((reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(y)) & 15) return -2;
  const long long threads = static_cast<long long>(n) * 32;
  rb::ec_combine_bwd_kernel<<<static_cast<int>((threads + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(dout), idx, gate, reinterpret_cast<const __nv_bfloat16*>(y),
      reinterpret_cast<__nv_bfloat16*>(dy), dgate, n, T, d);
  return static_cast<int>(cudaGetLastError());
}
