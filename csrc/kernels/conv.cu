// Direct 2-D convolution forward for small filter banks (the image-model front ends and the reference's conv2d
// workloads: 1-3 input channels, 8-32 filters of 3 x 3).  One thread owns one output pixel for eight output channels:
// every input tap is read once (coalesced along the image row) and used eight times against filters held in shared
// memory, the bias add and the NCHW store are part of the same kernel.  At these sizes the im2col matrix has a
// contraction of 9-27: padding it to a tensor-core tile and materialising it costs more than the arithmetic, which is
// why this shape class runs on the CUDA cores.  Larger banks take the im2col + tcgen05 GEMM path (nn/conv.py).
// The reference convolves with nested host loops over one input channel (crates/nn/src/conv.rs:88-215).
#include "conv.h"

#include "rb_common.cuh"

namespace rb {

constexpr int kConvOcPerThread = 8;
constexpr int kConvMaxFilterElems = 12288;

__global__ void __launch_bounds__(256)
conv2d_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
                  __nv_bfloat16* __restrict__ y, int N, int C, int H, int W, int O, int kh, int kw, int stride, int pad_h,
                  int pad_w, int Ho, int Wo) {
  extern __shared__ float w_sh[];                    // [O][C * kh * kw] fp32
  const int taps = C * kh * kw;
  for (int i = threadIdx.x; i < O * taps; i += blockDim.x) w_sh[i] = __bfloat162float(w[i]);
  __syncthreads();
  const long long pixels = static_cast<long long>(N) * Ho * Wo;
  const long long p = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (p >= pixels) return;
  const int wo = static_cast<int>(p % Wo);
  const long long t = p / Wo;
  const int ho = static_cast<int>(t % Ho);
  const int n = static_cast<int>(t / Ho);
  const int o0 = blockIdx.y * kConvOcPerThread;
  float acc[kConvOcPerThread];
#pragma unroll
  for (int j = 0; j < kConvOcPerThread; ++j)
    acc[j] = (bias != nullptr && o0 + j < O) ? __bfloat162float(bias[o0 + j]) : 0.f;
  const int hi0 = ho * stride - pad_h, wi0 = wo * stride - pad_w;
  int tap = 0;
  for (int c = 0; c < C; ++c) {
    const __nv_bfloat16* xc = x + (static_cast<long long>(n) * C + c) * H * W;
    for (int i = 0; i < kh; ++i) {
      const int hi = hi0 + i;
      const bool row_ok = hi >= 0 && hi < H;
      for (int j = 0; j < kw; ++j, ++tap) {
        const int wi = wi0 + j;
        if (!row_ok || wi < 0 || wi >= W) continue;
        const float v = __bfloat162float(xc[static_cast<long long>(hi) * W + wi]);
#pragma unroll
        for (int q = 0; q < kConvOcPerThread; ++q)
          if (o0 + q < O) acc[q] += v * w_sh[(o0 + q) * taps + tap];
      }
    }
  }
#pragma unroll
  for (int q = 0; q < kConvOcPerThread; ++q)
    if (o0 + q < O) y[((static_cast<long long>(n) * O + o0 + q) * Ho + ho) * Wo + wo] = __float2bfloat16(acc[q]);
}

}  // namespace rb

RB_API int rb_conv2d_fwd(const void* x, const void* w, const void* bias, void* y, int N, int C, int H, int W, int O, int kh,
                         int kw, int stride, int pad_h, int pad_w, void* stream) {
  if (!x || !w || !y || N <= 0 || C <= 0 || H <= 0 || W <= 0 || O <= 0 || kh <= 0 || kw <= 0 || stride <= 0 || pad_h < 0 ||
      pad_w < 0)
    return -1;
  const int Ho = (H + 2 * pad_h - kh) / stride + 1, Wo = (W + 2 * pad_w - kw) / stride + 1;
  if (Ho <= 0 || Wo <= 0) return -2;
  const long long taps = static_cast<long long>(C) * kh * kw;
  if (static_cast<long long>(O) * taps > rb::kConvMaxFilterElems) return -3;
  const long long pixels = static_cast<long long>(N) * Ho * Wo;
  const long long blocks = (pixels + 255) / 256;
  if (blocks > 0x7fffffffLL) return -1;
  const dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>((O + rb::kConvOcPerThread - 1) / rb::kConvOcPerThread));
  const size_t smem = static_cast<size_t>(O) * taps * sizeof(float);
  rb::conv2d_fwd_kernel<<<grid, 256, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),
      reinterpret_cast<const __nv_bfloat16*>(bias), reinterpret_cast<__nv_bfloat16*>(y), N, C, H, W, O, kh, kw, stride, pad_h,
      pad_w, Ho, Wo);
  return static_cast<int>(cudaGetLastError());
}
