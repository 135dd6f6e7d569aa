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

// ------------------------------------------------------------------------------------------------------------------
// Training path (and large filter banks): convolution as one GEMM over unfolded patches.
//   rb_im2col        x [N, C, H, W] -> cols [N * Ho * Wo, Kp]: row (n, ho, wo), column (c, i, j) = the tap's pixel or zero;
//                    columns [C * kh * kw, Kp) are zero padding so that rows have a 16-byte pitch for TMA
//   rb_col2im        the adjoint: dx[n, c, h, w] = sum of dcols over the (row, column) pairs that read that pixel, as a
//                    gather per pixel in a fixed order (no atomics)
//   rb_nhwc_to_nchw  y2 [N * L, ld] (first O columns) -> y [N, O, L]         (the GEMM's output into the layer's layout)
//   rb_nchw_to_nhwc  dy [N, O, L] -> dy2 [N * L, Op] with zero columns [O, Op) (the layer's gradient into the GEMM's layout)
// ------------------------------------------------------------------------------------------------------------------
namespace rb {

__global__ void __launch_bounds__(256)
im2col_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ cols, int N, int C, int H, int W, int kh, int kw,
              int stride, int pad_h, int pad_w, int Ho, int Wo, int Kp) {
  const long long total = static_cast<long long>(N) * Ho * Wo * Kp;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  const int K = C * kh * kw;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const int k = static_cast<int>(i % Kp);
    const long long row = i / Kp;
    __nv_bfloat16 v = __float2bfloat16(0.f);
    if (k < K) {
      const int wo = static_cast<int>(row % Wo), ho = static_cast<int>((row / Wo) % Ho), n = static_cast<int>(row / (static_cast<long long>(Wo) * Ho));
      const int j = k % kw, ii = (k / kw) % kh, c = k / (kw * kh);
      const int h = ho * stride - pad_h + ii, w = wo * stride - pad_w + j;
      if (h >= 0 && h < H && w >= 0 && w < W) v = x[((static_cast<long long>(n) * C + c) * H + h) * W + w];
    }
    cols[i] = v;
  }
}

__global__ void __launch_bounds__(256)
col2im_kernel(const __nv_bfloat16* __restrict__ dcols, __nv_bfloat16* __restrict__ dx, int N, int C, int H, int W, int kh, int kw,
              int stride, int pad_h, int pad_w, int Ho, int Wo, int Kp) {
  const long long total = static_cast<long long>(N) * C * H * W;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const int w = static_cast<int>(i % W), h = static_cast<int>((i / W) % H), c = static_cast<int>((i / (static_cast<long long>(W) * H)) % C);
    const int n = static_cast<int>(i / (static_cast<long long>(W) * H * C));
    float acc = 0.f;
    for (int ii = 0; ii < kh; ++ii) {
      const int hn = h + pad_h - ii;
      if (hn < 0 || hn % stride) continue;
      const int ho = hn / stride;
      if (ho >= Ho) continue;
      for (int j = 0; j < kw; ++j) {
        const int wn = w + pad_w - j;
        if (wn < 0 || wn % stride) continue;
        const int wo = wn / stride;
        if (wo >= Wo) continue;
        const long long row = (static_cast<long long>(n) * Ho + ho) * Wo + wo;
        acc += __bfloat162float(dcols[row * Kp + (c * kh + ii) * kw + j]);
      }
    }
    dx[i] = __float2bfloat16(acc);
  }
}

// 32 x 32 tiles through shared memory: both sides are read and written along their contiguous dimension
__global__ void __launch_bounds__(256)
nhwc_nchw_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, int L, int O, long long ld_src,
                 long long ld_dst_rows, int to_nchw) {
  // to_nchw: src [n][l][o] (pitch ld_src) -> dst [n][o][l];   else: src [n][o][l] -> dst [n][l][o] (pitch ld_dst_rows, zero fill)
  __shared__ __nv_bfloat16 tile[32][33];
  const int n = blockIdx.z;
  const int l0 = blockIdx.x * 32, o0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;          // 32 x 8
  if (to_nchw) {
    for (int r = ty; r < 32; r += 8) {
      const int l = l0 + r, o = o0 + tx;
      tile[r][tx] = (l < L && o < O) ? src[(static_cast<long long>(n) * L + l) * ld_src + o] : __float2bfloat16(0.f);
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
      const int o = o0 + r, l = l0 + tx;
      if (o < O && l < L) dst[(static_cast<long long>(n) * O + o) * L + l] = tile[tx][r];
    }
  } else {
    const int Op = static_cast<int>(ld_dst_rows);
    for (int r = ty; r < 32; r += 8) {
      const int o = o0 + r, l = l0 + tx;
      tile[r][tx] = (o < O && l < L) ? src[(static_cast<long long>(n) * O + o) * L + l] : __float2bfloat16(0.f);
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
      const int l = l0 + r, o = o0 + tx;
      if (l < L && o < Op) dst[(static_cast<long long>(n) * L + l) * Op + o] = tile[tx][r];
    }
  }
}

}  // namespace rb

namespace {
inline int conv_out(int size, int pad, int k, int stride) { return (size + 2 * pad - k) / stride + 1; }
inline int conv_grid(long long total) { long long b = (total + 255) / 256; return static_cast<int>(b < 148 * 16 ? (b > 0 ? b : 1) : 148 * 16); }
}  // namespace

RB_API int rb_im2col(const void* x, void* cols, int N, int C, int H, int W, int kh, int kw, int stride, int pad_h, int pad_w, int Kp,
                     void* stream) {
  if (!x || !cols || N <= 0 || C <= 0 || H <= 0 || W <= 0 || kh <= 0 || kw <= 0 || stride <= 0 || pad_h < 0 || pad_w < 0 || Kp < C * kh * kw) return -1;
  const int Ho = conv_out(H, pad_h, kh, stride), Wo = conv_out(W, pad_w, kw, stride);
  if (Ho <= 0 || Wo <= 0) return -1;
  const long long total = static_cast<long long>(N) * Ho * Wo * Kp;
  rb::im2col_kernel<<<conv_grid(total), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(cols), N, C, H, W, kh, kw, stride, pad_h, pad_w, Ho, Wo, Kp);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_col2im(const void* dcols, void* dx, int N, int C, int H, int W, int kh, int kw, int stride, int pad_h, int pad_w, int Kp,
                     void* stream) {
  if (!dcols || !dx || N <= 0 || C <= 0 || H <= 0 || W <= 0 || kh <= 0 || kw <= 0 || stride <= 0 || pad_h < 0 || pad_w < 0 || Kp < C * kh * kw) return -1;
  const int Ho = conv_out(H, pad_h, kh, stride), Wo = conv_out(W, pad_w, kw, stride);
  if (Ho <= 0 || Wo <= 0) return -1;
  const long long total = static_cast<long long>(N) * C * H * W;
  rb::col2im_kernel<<<conv_grid(total), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(dcols), reinterpret_cast<__nv_bfloat16*>(dx), N, C, H, W, kh, kw, stride, pad_h, pad_w, Ho, Wo, Kp);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_nhwc_to_nchw(const void* src, long long ld_src, void* dst, int N, int L, int O, void* stream) {
  if (!src || !dst || N <= 0 || L <= 0 || O <= 0 || ld_src < O || N > 65535) return -1;
  dim3 grid((L + 31) / 32, (O + 31) / 32, N);
  if (grid.y > 65535) return -1;
  rb::nhwc_nchw_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), reinterpret_cast<__nv_bfloat16*>(dst), L, O, ld_src, 0, 1);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_nchw_to_nhwc(const void* src, void* dst, int N, int L, int O, int Op, void* stream) {
  if (!src || !dst || N <= 0 || L <= 0 || O <= 0 || Op < O || N > 65535) return -1;
  dim3 grid((L + 31) / 32, (Op + 31) / 32, N);
  if (grid.y > 65535) return -1;
  rb::nhwc_nchw_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), reinterpret_cast<__nv_bfloat16*>(dst), L, O, 0, Op, 0);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------------------------
// Max pooling (crates/nn/src/conv.rs:228-340 pools on the host).  Forward writes the window maximum and the flat index
// (h * W + w) of the element that produced it (first maximum in row-major window order); backward is a gather per input
// element over the windows that contain it, so overlapping windows (stride < kernel) need no atomics.
// ------------------------------------------------------------------------------------------------------------------
namespace rb {

template <typename T> __device__ __forceinline__ float pool_ld(const T* p);
template <> __device__ __forceinline__ float pool_ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float pool_ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void pool_st(T* p, float v);
template <> __device__ __forceinline__ void pool_st<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void pool_st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

template <typename T>
__global__ void __launch_bounds__(256)
max_pool2d_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int* __restrict__ idx, long long planes, int H, int W, int k,
                      int stride, int Ho, int Wo) {
  const long long total = planes * Ho * Wo;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const int wo = static_cast<int>(i % Wo), ho = static_cast<int>((i / Wo) % Ho);
    const long long pl = i / (static_cast<long long>(Wo) * Ho);
    const T* xp = x + pl * H * W;
    float best = -INFINITY;
    int arg = (ho * stride) * W + wo * stride;
    for (int a = 0; a < k; ++a) {
      const int h = ho * stride + a;
      if (h >= H) break;
      for (int b = 0; b < k; ++b) {
        const int w = wo * stride + b;
        if (w >= W) break;
        const float v = pool_ld(xp + h * W + w);
        if (v > best || (v != v && best == best)) { best = v; arg = h * W + w; }      // NaN wins, like the reference math
      }
    }
    pool_st(y + i, best);
    idx[i] = arg;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
max_pool2d_bwd_kernel(const T* __restrict__ dy, const int* __restrict__ idx, T* __restrict__ dx, long long planes, int H, int W,
                      int k, int stride, int Ho, int Wo) {
  const long long total = planes * H * W;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const int w = static_cast<int>(i % W), h = static_cast<int>((i / W) % H);
    const long long pl = i / (static_cast<long long>(W) * H);
    const int me = h * W + w;
    // windows (ho, wo) with ho * stride <= h < ho * stride + k
    const int ho_hi = min(Ho - 1, h / stride), wo_hi = min(Wo - 1, w / stride);
    const int ho_lo = max(0, (h - k + stride) / stride), wo_lo = max(0, (w - k + stride) / stride);
    float acc = 0.f;
    for (int ho = ho_lo; ho <= ho_hi; ++ho)
      for (int wo = wo_lo; wo <= wo_hi; ++wo) {
        const long long o = (pl * Ho + ho) * Wo + wo;
        if (idx[o] == me) acc += pool_ld(dy + o);
      }
    pool_st(dx + i, acc);
  }
}

}  // namespace rb

RB_API int rb_max_pool2d_fwd(const void* x, void* y, int* idx, long long planes, int H, int W, int k, int stride, int is_bf16,
                             void* stream) {
  if (!x || !y || !idx || planes <= 0 || H <= 0 || W <= 0 || k <= 0 || stride <= 0 || k > H || k > W) return -1;
  const int Ho = (H - k) / stride + 1, Wo = (W - k) / stride + 1;
  const long long total = planes * Ho * Wo;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (is_bf16)
    rb::max_pool2d_fwd_kernel<__nv_bfloat16><<<conv_grid(total), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                                              reinterpret_cast<__nv_bfloat16*>(y), idx, planes, H, W, k, stride, Ho, Wo);
  else
    rb::max_pool2d_fwd_kernel<float><<<conv_grid(total), 256, 0, s>>>(reinterpret_cast<const float*>(x), reinterpret_cast<float*>(y), idx,
                                                                      planes, H, W, k, stride, Ho, Wo);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_max_pool2d_bwd(const void* dy, const int* idx, void* dx, long long planes, int H, int W, int k, int stride, int is_bf16,
                             void* stream) {
  if (!dy || !dx || !idx || planes <= 0 || H <= 0 || W <= 0 || k <= 0 || stride <= 0 || k > H || k > W) return -1;
  const int Ho = (H - k) / stride + 1, Wo = (W - k) / stride + 1;
  const long long total = planes * H * W;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (is_bf16)
    rb::max_pool2d_bwd_kernel<__nv_bfloat16><<<conv_grid(total), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(dy), idx,
                                                                              reinterpret_cast<__nv_bfloat16*>(dx), planes, H, W, k, stride, Ho, Wo);
  else
    rb::max_pool2d_bwd_kernel<float><<<conv_grid(total), 256, 0, s>>>(reinterpret_cast<const float*>(dy), idx, reinterpret_cast<float*>(dx),
                                                                      planes, H, W, k, stride, Ho, Wo);
  return static_cast<int>(cudaGetLastError());
}
