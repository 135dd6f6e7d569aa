// Rotary position embedding (theta configurable, 500000 for the Llama-style 8B config) and the SwiGLU
// gate.  Both are bandwidth-bound single-pass kernels with 128-bit accesses.  Neither exists in the
// reference (its "SwiGLU-style" expert multiplies gate and up without the SiLU,
// crates/nn/src/shared_expert.rs:143-169); they are required by its Llama-shaped benchmark config.
#include "rope.h"

#include "rb_common.cuh"

namespace rb {

// one thread handles 8 consecutive pair indices i..i+7 of one (token, head): loads x[i..i+7] and x[i+half..]
__global__ void __launch_bounds__(256)
rope_kernel(__nv_bfloat16* __restrict__ x, long long ld, const long long* __restrict__ positions, long long tokens,
            int heads, int head_dim, int seq_len, long long pos_offset, float log2_theta, int inverse) {
  const int half = head_dim / 2;
  const int groups = half / 8;
  const long long total = tokens * heads * groups;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int gidx = static_cast<int>(i % groups);
    const long long th = i / groups;
    const int h = static_cast<int>(th % heads);
    const long long t = th / heads;
    const float pos = static_cast<float>(positions ? positions[t] : pos_offset + (t % seq_len));
    __nv_bfloat16* p = x + t * ld + static_cast<long long>(h) * head_dim + gidx * 8;
    uint4 lo = *reinterpret_cast<uint4*>(p), hi = *reinterpret_cast<uint4*>(p + half);
    uint32_t* pl = reinterpret_cast<uint32_t*>(&lo);
    uint32_t* ph = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16x2(pl[j]), b = unpack_bf16x2(ph[j]);
      float r0[2] = {a.x, a.y}, r1[2] = {b.x, b.y};
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int idx = gidx * 8 + j * 2 + e;
        // inv_freq = theta^(-2*idx/head_dim)
        const float inv_freq = exp2f(-log2_theta * (2.f * idx) / static_cast<float>(head_dim));
        float s, c;
        sincosf(pos * inv_freq, &s, &c);
        if (inverse) s = -s;
        const float x0 = r0[e], x1 = r1[e];
        r0[e] = x0 * c - x1 * s;
        r1[e] = x1 * c + x0 * s;
      }
      pl[j] = pack_bf16x2(r0[0], r0[1]);
      ph[j] = pack_bf16x2(r1[0], r1[1]);
    }
    *reinterpret_cast<uint4*>(p) = lo;
    *reinterpret_cast<uint4*>(p + half) = hi;
  }
}

__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, long long ld_gu, __nv_bfloat16* __restrict__ h, long long ld_h,
                  long long tokens, int F) {
  const int chunks = F / 8;
  const long long total = tokens * chunks;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long t = i / chunks;
    const int c = static_cast<int>(i - t * chunks) * 8;
    uint4 g = *reinterpret_cast<const uint4*>(gu + t * ld_gu + c);
    uint4 u = *reinterpret_cast<const uint4*>(gu + t * ld_gu + F + c);
    uint4 o;
    const uint32_t* pg = reinterpret_cast<const uint32_t*>(&g);
    const uint32_t* pu = reinterpret_cast<const uint32_t*>(&u);
    uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(pg[j]), b = unpack_bf16x2(pu[j]);
      po[j] = pack_bf16x2(silu(a.x) * b.x, silu(a.y) * b.y);
    }
    *reinterpret_cast<uint4*>(h + t * ld_h + c) = o;
  }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dh, long long ld_dh, const __nv_bfloat16* __restrict__ gu,
                  long long ld_gu, __nv_bfloat16* __restrict__ dgu, long long ld_dgu, long long tokens, int F) {
  const int chunks = F / 8;
  const long long total = tokens * chunks;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long t = i / chunks;
    const int c = static_cast<int>(i - t * chunks) * 8;
    uint4 g = *reinterpret_cast<const uint4*>(gu + t * ld_gu + c);
    uint4 u = *reinterpret_cast<const uint4*>(gu + t * ld_gu + F + c);
    uint4 d = *reinterpret_cast<const uint4*>(dh + t * ld_dh + c);
    uint4 og, ou;
    const uint32_t* pg = reinterpret_cast<const uint32_t*>(&g);
    const uint32_t* pu = reinterpret_cast<const uint32_t*>(&u);
    const uint32_t* pd = reinterpret_cast<const uint32_t*>(&d);
    uint32_t* qg = reinterpret_cast<uint32_t*>(&og);
    uint32_t* qu = reinterpret_cast<uint32_t*>(&ou);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(pg[j]), b = unpack_bf16x2(pu[j]), e = unpack_bf16x2(pd[j]);
      qg[j] = pack_bf16x2(e.x * b.x * silu_grad(a.x), e.y * b.y * silu_grad(a.y));
      qu[j] = pack_bf16x2(e.x * silu(a.x), e.y * silu(a.y));
    }
    *reinterpret_cast<uint4*>(dgu + t * ld_dgu + c) = og;
    *reinterpret_cast<uint4*>(dgu + t * ld_dgu + F + c) = ou;
  }
}

inline int grid1d(long long n) {
  long long b = (n + 255) / 256;
  if (b > 148LL * 16) b = 148LL * 16;
  return static_cast<int>(b < 1 ? 1 : b);
}

}  // namespace rb

RB_API int rb_rope(void* x, long long ld, const long long* positions, long long tokens, int heads, int head_dim,
                   int seq_len, long long pos_offset, float theta, int inverse, void* stream_v) {
  if (tokens <= 0 || heads <= 0 || head_dim <= 0 || (head_dim % 16) || (ld % 8) || theta <= 0.f) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (!positions && seq_len <= 0)) return -2;
  const long long total = tokens * heads * (head_dim / 16);
  rb::rope_kernel<<<rb::grid1d(total), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<__nv_bfloat16*>(x), ld, positions, tokens, heads, head_dim, seq_len < 1 ? 1 : seq_len, pos_offset,
      log2f(theta), inverse);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_swiglu_fwd(const void* gu, long long ld_gu, void* h, long long ld_h, long long tokens, int F, void* stream_v) {
  if (tokens <= 0 || F <= 0 || (F % 8) || (ld_gu % 8) || (ld_h % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(h)) & 15) return -2;
  rb::swiglu_fwd_kernel<<<rb::grid1d(tokens * (F / 8)), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const __nv_bfloat16*>(gu), ld_gu, reinterpret_cast<__nv_bfloat16*>(h), ld_h, tokens, F);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_swiglu_bwd(const void* dh, long long ld_dh, const void* gu, long long ld_gu, void* dgu, long long ld_dgu,
                         long long tokens, int F, void* stream_v) {
  if (tokens <= 0 || F <= 0 || (F % 8) || (ld_gu % 8) || (ld_dh % 8) || (ld_dgu % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(dh) | reinterpret_cast<uintptr_t>(dgu)) & 15) return -2;
  rb::swiglu_bwd_kernel<<<rb::grid1d(tokens * (F / 8)), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const __nv_bfloat16*>(dh), ld_dh, reinterpret_cast<const __nv_bfloat16*>(gu), ld_gu,
      reinterpret_cast<__nv_bfloat16*>(dgu), ld_dgu, tokens, F);
  return static_cast<int>(cudaGetLastError());
}
