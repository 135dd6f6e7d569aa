// Softmax-cross-entropy over large vocabularies, fused forward + backward, and the plain row
// softmax / log-softmax pair.
//
// One CTA per row.  The row is streamed twice: an online (max, sum-exp) pass, then a pass that
// writes (softmax - onehot) * scale.  The second read of a 100 KB bf16 row comes out of L2.
// Replaces the reference's cross_entropy_loss tape op, which builds one-hot targets on the host
// (crates/autodiff/src/lib.rs:645-806), the global-log-softmax CrossEntropyLoss
// (crates/nn/src/loss.rs:82-114) and the O(classes^2) WGSL softmax (shaders.wgsl:743-803).
#include "loss.h"

#include <float.h>

#include "rb_common.cuh"

namespace rb {

constexpr int kCeThreads = 512;

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  if (mm == -INFINITY) { m = mm; s = 0.f; return; }
  s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
  m = mm;
}

__device__ __forceinline__ void block_online_reduce(float& m, float& s, float* sh_m, float* sh_s) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  if (lane == 0) { sh_m[warp] = m; sh_s[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    m = lane < nwarps ? sh_m[lane] : -INFINITY;
    s = lane < nwarps ? sh_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_merge(m, s, m2, s2);
    }
    if (lane == 0) { sh_m[0] = m; sh_s[0] = s; }
  }
  __syncthreads();
  m = sh_m[0];
  s = sh_s[0];
}

__global__ void __launch_bounds__(kCeThreads)
cross_entropy_kernel(const __nv_bfloat16* logits, long long ld, const long long* __restrict__ targets,
                     float* __restrict__ loss, float* __restrict__ lse_out, __nv_bfloat16* dlogits, long long ldd,
                     int n_valid, int n_pad, float grad_scale, long long ignore_index RB_BOUNDS_PARAM) {
  __shared__ float sh_m[32], sh_s[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* x = logits + row * ld;
  const long long tgt = targets[row];
  const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= n_valid;
  if (ignored && tgt != ignore_index && threadIdx.x == 0) RB_BOUNDS_HIT(105);     // not a class and not the ignore marker
  // `dlogits` may be the same memory as `logits` (the gradient overwrites the logits): the target logit is read
  // here, before the reduction's barriers, because other warps start storing gradients right after them; and the
  // row is read with plain loads, not through the read-only path.
  float x_tgt = 0.f;
  if (threadIdx.x == 0 && !ignored) x_tgt = __bfloat162float(x[tgt]);
  const bool vec_ok = ((ld & 7) == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  float m = -INFINITY, s = 0.f;
  const int n8 = vec_ok ? (n_valid / 8) : 0;
  for (int i = threadIdx.x; i < n8; i += blockDim.x) {
    uint4 u = reinterpret_cast<const uint4*>(x)[i];
    float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
    const float lm = fmaxf(fmaxf(fmaxf(f0.x, f0.y), fmaxf(f1.x, f1.y)), fmaxf(fmaxf(f2.x, f2.y), fmaxf(f3.x, f3.y)));
    const float mm = fmaxf(m, lm);
    s = s * __expf(m - mm) + __expf(f0.x - mm) + __expf(f0.y - mm) + __expf(f1.x - mm) + __expf(f1.y - mm) +
        __expf(f2.x - mm) + __expf(f2.y - mm) + __expf(f3.x - mm) + __expf(f3.y - mm);
    m = mm;
  }
  for (int i = n8 * 8 + threadIdx.x; i < n_valid; i += blockDim.x) {
    const float v = __bfloat162float(x[i]);
    const float mm = fmaxf(m, v);
    s = s * __expf(m - mm) + __expf(v - mm);
    m = mm;
  }
  block_online_reduce(m, s, sh_m, sh_s);
  const float lse = m + logf(s);
  if (threadIdx.x == 0) {
    if (lse_out) lse_out[row] = lse;
    loss[row] = ignored ? 0.f : lse - x_tgt;
  }
  if (dlogits == nullptr) return;
  __nv_bfloat16* dx = dlogits + row * ldd;
  const float gs = ignored ? 0.f : grad_scale;
  const bool vec_out = vec_ok && ((ldd & 7) == 0) && ((reinterpret_cast<uintptr_t>(dlogits) & 15) == 0);
  const int np8 = vec_out ? (n_pad / 8) : 0;
  for (int i = threadIdx.x; i < np8; i += blockDim.x) {
    const int c0 = i * 8;
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (c0 < n_valid) {
      float f[8];
      if (c0 + 8 <= n_valid) {
        uint4 u = reinterpret_cast<const uint4*>(x)[i];
        float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
        f[0] = f0.x; f[1] = f0.y; f[2] = f1.x; f[3] = f1.y; f[4] = f2.x; f[5] = f2.y; f[6] = f3.x; f[7] = f3.y;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = (c0 + j < n_valid) ? __bfloat162float(x[c0 + j]) : -INFINITY;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float p = (c0 + j < n_valid) ? __expf(f[j] - lse) : 0.f;
        if (c0 + j == tgt) p -= 1.f;
        f[j] = p * gs;
      }
      o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
      o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
    }
    reinterpret_cast<uint4*>(dx)[i] = o;
  }
  for (int i = np8 * 8 + threadIdx.x; i < n_pad; i += blockDim.x) {
    float p = 0.f;
    if (i < n_valid) {
      p = __expf(__bfloat162float(x[i]) - lse);
      if (i == tgt) p -= 1.f;
      p *= gs;
    }
    dx[i] = __float2bfloat16(p);
  }
}

template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st_from_float(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_from_float(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

template <typename T>
__global__ void __launch_bounds__(256)
softmax_rows_kernel(const T* __restrict__ x, T* __restrict__ y, int n, long long ldx, long long ldy, int log_mode) {
  __shared__ float sh_m[32], sh_s[32];
  const long long row = blockIdx.x;
  const T* xr = x + row * ldx;
  T* yr = y + row * ldy;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = ld_as_float(xr + i);
    const float mm = fmaxf(m, v);
    s = s * __expf(m - mm) + __expf(v - mm);
    m = mm;
  }
  block_online_reduce(m, s, sh_m, sh_s);
  const float lse = m + logf(s);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = ld_as_float(xr + i) - lse;
    st_from_float(yr + i, log_mode ? v : expf(v));
  }
}

// softmax:     dx = y * (dy - sum(dy * y));   log-softmax: dx = dy - exp(y) * sum(dy)
__global__ void __launch_bounds__(256)
softmax_rows_bwd_kernel(const float* __restrict__ out, const float* __restrict__ dy, float* __restrict__ dx, int n,
                        int log_mode) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const float* o = out + row * n;
  const float* g = dy + row * n;
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += log_mode ? g[i] : g[i] * o[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) sh[0] = v;
  }
  __syncthreads();
  const float tot = sh[0];
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    dx[row * n + i] = log_mode ? g[i] - expf(o[i]) * tot : o[i] * (g[i] - tot);
}

}  // namespace rb

namespace rb {
__global__ void __launch_bounds__(256)
ce_grad_lse_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, const long long* __restrict__ targets,
                   const float* __restrict__ lse, __nv_bfloat16* __restrict__ dlogits, long long ldd, int rows, int n,
                   float grad_scale) {
  const int c8 = n / 8;
  const long long total = static_cast<long long>(rows) * c8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / c8;
    const int c = static_cast<int>(i - r * c8) * 8;
    const float l = __ldg(lse + r);
    const long long t = __ldg(targets + r);
    const uint4 u = *reinterpret_cast<const uint4*>(logits + r * ld + c);
    const uint32_t* pu = reinterpret_cast<const uint32_t*>(&u);
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(pu[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = (__expf(v[j] - l) - ((c + j) == t ? 1.f : 0.f)) * grad_scale;
    uint4 o;
    o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]); o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(dlogits + r * ldd + c) = o;
  }
}
}  // namespace rb

RB_API int rb_cross_entropy_grad_lse(const void* logits, long long ld, const long long* targets, const float* lse,
                                     void* dlogits, long long ldd, int rows, int n, float grad_scale, void* stream_v) {
  if (rows <= 0 || n <= 0) return 0;
  if (!logits || !targets || !lse || !dlogits || (n % 8) || (ld % 8) || (ldd % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(dlogits)) & 15) return -2;
  const long long total = static_cast<long long>(rows) * (n / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  rb::ce_grad_lse_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const __nv_bfloat16*>(logits), ld, targets, lse, reinterpret_cast<__nv_bfloat16*>(dlogits), ldd,
      rows, n, grad_scale);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_cross_entropy(const void* logits, long long ld, const long long* targets, float* loss, float* lse,
                            void* dlogits, long long ldd, int rows, int n_valid, int n_pad, float grad_scale,
                            long long ignore_index, void* stream_v) {
  if (rows <= 0 || n_valid <= 0 || n_pad < n_valid || !logits || !targets || !loss) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  rb::cross_entropy_kernel<<<rows, rb::kCeThreads, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(logits), ld, targets, loss, lse, reinterpret_cast<__nv_bfloat16*>(dlogits),
      ldd, n_valid, n_pad, grad_scale, ignore_index RB_BOUNDS_ARG);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_softmax_rows(const void* x, void* y, int rows, int n, long long ldx, long long ldy, int log_mode,
                           int dtype, void* stream_v) {
  if (rows <= 0 || n <= 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (dtype == 0)
    rb::softmax_rows_kernel<float><<<rows, 256, 0, stream>>>(reinterpret_cast<const float*>(x),
                                                             reinterpret_cast<float*>(y), n, ldx, ldy, log_mode);
  else
    rb::softmax_rows_kernel<__nv_bfloat16><<<rows, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                                     reinterpret_cast<__nv_bfloat16*>(y), n, ldx, ldy,
                                                                     log_mode);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_softmax_rows_bwd(const float* out, const float* dy, float* dx, int rows, int n, int log_mode,
                               void* stream_v) {
  if (rows <= 0 || n <= 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  rb::softmax_rows_bwd_kernel<<<rows, 256, 0, stream>>>(out, dy, dx, n, log_mode);
  return static_cast<int>(cudaGetLastError());
}
