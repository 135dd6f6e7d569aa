// Quantisation kernels for the 8-bit / 4-bit linear layers (counterparts of the host loops in
// crates/nn/src/quantization.rs:97-160 quantize / dequantize and :324-430 group-wise int4).
//
//   rb_quantize_fp8_rows   bf16 [rows, n] -> e4m3 bytes [rows, n] + one fp32 scale per row (dynamic, absmax / 448).
//                          Feeds the A operand (tokens) or the B operand (weights, one scale per output channel) of
//                          the tcgen05 kind::f8f6f4 GEMM, which multiplies the scales back in its epilogue.
//   rb_dequant_int8_bf16   int8 [rows, n] (minus a zero point) -> bf16, exact: |q - z| <= 255 has 8 significant bits.
//                          The scale stays outside and goes into the GEMM epilogue.
//   rb_dequant_int4_bf16   packed nibbles [rows, n / 2] with one fp32 scale per (row, group) -> bf16 (q - 8) * scale.
//
// One warp per row for the fp8 quantiser (two passes over a row held in registers when it fits), grid-stride loops of
// 16-byte vectors for the dequantisers.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "quant.h"
#include "rb_common.cuh"

namespace rb {

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// kVecs: 16-byte vectors (8 bf16) a lane keeps in registers; rows longer than 32 * 8 * kVecs are read twice.
template <int kVecs>
__global__ void __launch_bounds__(256)
quantize_fp8_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ out, long long ldo,
                         float* __restrict__ scales, int rows, int n) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int nvec = n >> 3;                       // n is a multiple of 16
  for (int row = warp; row < rows; row += nwarps) {
    const uint4* xp = reinterpret_cast<const uint4*>(x + row * ldx);
    uint4 keep[kVecs];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < kVecs; ++i) {
      const int v = lane + i * 32;
      keep[i] = v < nvec ? __ldg(xp + v) : make_uint4(0, 0, 0, 0);
      const uint32_t w[4] = {keep[i].x, keep[i].y, keep[i].z, keep[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
    for (int v = lane + kVecs * 32; v < nvec; v += 32) {
      const uint4 q = __ldg(xp + v);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
    const float inv = __fdiv_rn(1.f, scale);      // elements are multiplied by the rounded reciprocal (the CPU path does the same)
    if (lane == 0) scales[row] = scale;
    uint2* op = reinterpret_cast<uint2*>(out + row * ldo);
    auto emit = [&](int v, const uint4& q) {
      const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
      uint2 o;
      o.x = pack_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
      o.y = pack_e4m3x4(c.x * inv, c.y * inv, d.x * inv, d.y * inv);
      op[v] = o;
    };
#pragma unroll
    for (int i = 0; i < kVecs; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) emit(v, keep[i]);
    }
    for (int v = lane + kVecs * 32; v < nvec; v += 32) emit(v, __ldg(xp + v));
  }
}

__global__ void __launch_bounds__(256)
dequant_int8_bf16_kernel(const int8_t* __restrict__ q, const float* __restrict__ zero_point, int zp_per_row,
                         __nv_bfloat16* __restrict__ out, int rows, int n) {
  const long long nvec = static_cast<long long>(rows) * n / 16;        // n is a multiple of 16
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(q) + i);
    const float z = zero_point ? __ldg(zero_point + (zp_per_row ? (i * 16) / n : 0)) : 0.f;
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float b0 = static_cast<float>(static_cast<int8_t>(w[j] & 0xff)) - z;
      const float b1 = static_cast<float>(static_cast<int8_t>((w[j] >> 8) & 0xff)) - z;
      const float b2 = static_cast<float>(static_cast<int8_t>((w[j] >> 16) & 0xff)) - z;
      const float b3 = static_cast<float>(static_cast<int8_t>(w[j] >> 24)) - z;
      o[2 * j] = pack_bf16x2(b0, b1);
      o[2 * j + 1] = pack_bf16x2(b2, b3);
    }
    uint4* op = reinterpret_cast<uint4*>(out) + 2 * i;
    op[0] = make_uint4(o[0], o[1], o[2], o[3]);
    op[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// Byte b of a row holds elements 2b (low nibble) and 2b + 1 (high nibble); a 16-byte vector is 32 elements, which never
// straddles a group (the group size is a multiple of 32).
__global__ void __launch_bounds__(256)
dequant_int4_bf16_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales, int group_size,
                         __nv_bfloat16* __restrict__ out, int rows, int n) {
  const int vec_per_row = n / 32, groups = n / group_size;
  const long long nvec = static_cast<long long>(rows) * vec_per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const long long row = i / vec_per_row;
    const int v = static_cast<int>(i - row * vec_per_row);
    const float s = __ldg(scales + row * groups + (v * 32) / group_size);
    const uint4 p = __ldg(reinterpret_cast<const uint4*>(packed) + i);
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
    uint4* op = reinterpret_cast<uint4*>(out + row * n + v * 32);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t o[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t byte = (w[j] >> (8 * b)) & 0xff;
        o[b] = pack_bf16x2((static_cast<float>(byte & 15u) - 8.f) * s, (static_cast<float>(byte >> 4) - 8.f) * s);
      }
      op[j] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

}  // namespace rb

RB_API int rb_quantize_fp8_rows(const void* x, long long ldx, void* out, long long ldo, void* scales, int rows, int n,
                                void* stream_v) {
  if (rows <= 0 || n <= 0) return -1;
  if ((n & 15) || (ldx & 7) || (ldo & 15) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return -2;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const int warps_per_block = 8;
  long long blocks = (static_cast<long long>(rows) + warps_per_block - 1) / warps_per_block;
  if (blocks > 148 * 16) blocks = 148 * 16;
  auto xp = reinterpret_cast<const __nv_bfloat16*>(x);
  auto op = reinterpret_cast<uint8_t*>(out);
  auto sp = reinterpret_cast<float*>(scales);
  if (n <= 32 * 8 * 4)
    rb::quantize_fp8_rows_kernel<4><<<static_cast<int>(blocks), 256, 0, stream>>>(xp, ldx, op, ldo, sp, rows, n);
  else
    rb::quantize_fp8_rows_kernel<16><<<static_cast<int>(blocks), 256, 0, stream>>>(xp, ldx, op, ldo, sp, rows, n);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_dequant_int8_bf16(const void* q, const void* zero_point, int zp_per_row, void* out, int rows, int n,
                                void* stream_v) {
  if (rows <= 0 || n <= 0) return -1;
  if ((n & 15) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return -2;
  const long long nvec = static_cast<long long>(rows) * n / 16;
  long long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  rb::dequant_int8_bf16_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const int8_t*>(q), reinterpret_cast<const float*>(zero_point), zp_per_row,
      reinterpret_cast<__nv_bfloat16*>(out), rows, n);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_dequant_int4_bf16(const void* packed, const void* scales, int group_size, void* out, int rows, int n,
                                void* stream_v) {
  if (rows <= 0 || n <= 0 || group_size <= 0) return -1;
  if ((n & 31) || (group_size & 31) || (n % group_size) || (reinterpret_cast<uintptr_t>(packed) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return -2;
  const long long nvec = static_cast<long long>(rows) * (n / 32);
  long long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  rb::dequant_int4_bf16_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const uint8_t*>(packed), reinterpret_cast<const float*>(scales), group_size,
      reinterpret_cast<__nv_bfloat16*>(out), rows, n);
  return static_cast<int>(cudaGetLastError());
}
