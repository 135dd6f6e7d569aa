// LayerNorm / RMSNorm forward and backward for bf16 activations with fp32 statistics.
//
// One, two or four warps own one row and keep it in registers (row length up to 8192), so every
// element is read from HBM exactly once per pass.  The backward pass produces dx and, through a partial
// buffer of one fp32 row per CTA, the parameter gradients; a second kernel folds the partials in a
// fixed order, which keeps dgamma/dbeta bit-reproducible from run to run.
//
// Semantics follow the reference's host-side LayerNorm: population variance, eps inside the square
// root (crates/nn/src/normalization.rs:87-158; backward crates/autodiff/src/lib.rs:1167-1214).
#include "norm.h"

#include "rb_common.cuh"

namespace rb {

constexpr int kNormWarps = 4;

__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = o;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
  v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y; v[4] = f2.x; v[5] = f2.y; v[6] = f3.x; v[7] = f3.y;
}

// A row is owned by WPR warps of the CTA (1, 2 or 4), each lane holding CHUNKS x 8 elements, so
// that rows up to 8192 wide stay in registers without spilling.
template <int WPR>
__device__ __forceinline__ float row_sum(float v, float* red, int warp) {
  v = warp_sum(v);
  if (WPR == 1) return v;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[warp] = v;
  __syncthreads();
  float s = 0.f;
  const int w0 = (warp / WPR) * WPR;
#pragma unroll
  for (int i = 0; i < WPR; ++i) s += red[w0 + i];
  return s;
}

template <int CHUNKS, int WPR>
__device__ __forceinline__ int col_of(int wr, int c, int lane) { return ((wr * CHUNKS + c) * 32 + lane) * 8; }

template <int CHUNKS, int WPR>
__device__ __forceinline__ void load_row(const __nv_bfloat16* p, int n, int wr, int lane, bool valid,
                                         float (&x)[CHUNKS][8]) {
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = col_of<CHUNKS, WPR>(wr, c, lane);
    if (valid && col < n) {
      load8(p + col, x[c]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[c][j] = 0.f;
    }
  }
}

// y = (x - mean) * rstd * gamma + beta        (rms: y = x * rstd * gamma)
template <int CHUNKS, int WPR, bool RMS>
__global__ void __launch_bounds__(kNormWarps * 32)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ gamma,
                const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y, long long ldy,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int n, float eps) {
  __shared__ float red[kNormWarps];
  constexpr int RPB = kNormWarps / WPR;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int wr = warp % WPR;
  const float inv_n = 1.f / static_cast<float>(n);
  for (long long base = static_cast<long long>(blockIdx.x) * RPB; base < rows;
       base += static_cast<long long>(gridDim.x) * RPB) {
    const long long row = base + warp / WPR;
    const bool valid = row < rows;
    float v[CHUNKS][8];
    load_row<CHUNKS, WPR>(x + row * ldx, n, wr, lane, valid, v);
    float mean = 0.f;
    if (!RMS) {
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int j = 0; j < 8; ++j) s += v[c][j];
      mean = row_sum<WPR>(s, red, warp) * inv_n;
    }
    float sq = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      if (col_of<CHUNKS, WPR>(wr, c, lane) < n) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = v[c][j] - mean;
          sq += d * d;
        }
      }
    }
    const float var = row_sum<WPR>(sq, red, warp) * inv_n;
    const float rstd = rsqrtf(var + eps);
    if (!valid) continue;
    if (lane == 0 && wr == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = col_of<CHUNKS, WPR>(wr, c, lane);
      if (col < n) {
        float g[8], b[8], o[8];
        load8(gamma + col, g);
        if (beta) load8(beta + col, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = (v[c][j] - mean) * rstd * g[j];
          if (beta) o[j] += b[j];
        }
        store8(y + row * ldy + col, o);
      }
    }
  }
}

// dx = rstd * (g*dy - mean(g*dy) - xhat * mean(g*dy*xhat))   (+ dres)
// rms: dx = rstd * (g*dy - xhat * mean(g*dy*xhat))
// Parameter gradients accumulate per row-slot in shared memory (each lane owns its columns), are
// folded over the row-slots of the CTA in a fixed order, and leave as one partial row per CTA:
// partial[blockIdx.x][0..n) = dgamma, partial[gridDim.x + blockIdx.x][0..n) = dbeta.
template <int CHUNKS, int WPR, bool RMS>
__global__ void __launch_bounds__(kNormWarps * 32)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, long long lddy, const __nv_bfloat16* __restrict__ x,
                long long ldx, const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres, long long lddres,
                __nv_bfloat16* __restrict__ dx, long long lddx, float* __restrict__ partial, int rows, int n) {
  extern __shared__ float sm[];   // [RPB][2][n_pad]
  __shared__ float red[kNormWarps];
  constexpr int RPB = kNormWarps / WPR;
  constexpr int n_pad = WPR * CHUNKS * 256;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int wr = warp % WPR;
  const int slot = warp / WPR;
  const float inv_n = 1.f / static_cast<float>(n);
  float* sg = sm + (slot * 2 + 0) * n_pad;
  float* sb = sm + (slot * 2 + 1) * n_pad;
  // A thread sees the same columns in every row it processes, so the dgamma / dbeta sums stay in registers
  // until the end of the walk.
  float ag[CHUNKS][8], ab[CHUNKS][8];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { ag[c][j] = 0.f; ab[c][j] = 0.f; }
  }

  // gamma is the same for every row: kept packed in registers
  uint4 gpk[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = col_of<CHUNKS, WPR>(wr, c, lane);
    gpk[c] = col < n ? *reinterpret_cast<const uint4*>(gamma + col) : make_uint4(0u, 0u, 0u, 0u);
  }
  // The three input rows (x, dy, residual-branch gradient) of the NEXT row this warp will process are requested
  // before the current row's reductions, packed as loaded: the kernel is bound by memory latency otherwise.
  uint4 nx[CHUNKS], ny[CHUNKS], nr[CHUNKS];
  float nmean = 0.f, nrstd = 0.f;
  auto fetch = [&](long long row) {
    const bool valid = row < rows;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = col_of<CHUNKS, WPR>(wr, c, lane);
      const bool in = valid && col < n;
      nx[c] = in ? *reinterpret_cast<const uint4*>(x + row * ldx + col) : make_uint4(0u, 0u, 0u, 0u);
      ny[c] = in ? *reinterpret_cast<const uint4*>(dy + row * lddy + col) : make_uint4(0u, 0u, 0u, 0u);
      nr[c] = (in && dres) ? *reinterpret_cast<const uint4*>(dres + row * lddres + col) : make_uint4(0u, 0u, 0u, 0u);
    }
    nmean = (RMS || !valid) ? 0.f : mean_in[row];
    nrstd = valid ? rstd_in[row] : 0.f;
  };
  auto unpack8 = [](const uint4& u, float (&v)[8]) {
    const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
    v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y; v[4] = f2.x; v[5] = f2.y; v[6] = f3.x; v[7] = f3.y;
  };
  const long long step = static_cast<long long>(gridDim.x) * RPB;
  fetch(static_cast<long long>(blockIdx.x) * RPB + slot);
  for (long long base = static_cast<long long>(blockIdx.x) * RPB; base < rows; base += step) {
    const long long row = base + slot;
    const bool valid = row < rows;
    float xv[CHUNKS][8], gy[CHUNKS][8];
    uint4 rpk[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      unpack8(nx[c], xv[c]);
      unpack8(ny[c], gy[c]);
      rpk[c] = nr[c];
    }
    const float mean = nmean, rstd = nrstd;
    if (base + step < rows) fetch(row + step);          // every warp of the CTA takes this branch together
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = col_of<CHUNKS, WPR>(wr, c, lane);
      if (valid && col < n) {
        float g[8];
        unpack8(gpk[c], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xhat = (xv[c][j] - mean) * rstd;
          const float d = gy[c][j];
          ag[c][j] = fmaf(d, xhat, ag[c][j]);
          ab[c][j] += d;
          const float gd = d * g[j];
          xv[c][j] = xhat;
          gy[c][j] = gd;
          s1 += gd;
          s2 += gd * xhat;
        }
      }
    }
    s1 = RMS ? 0.f : row_sum<WPR>(s1, red, warp) * inv_n;
    s2 = row_sum<WPR>(s2, red, warp) * inv_n;
    if (!valid) continue;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = col_of<CHUNKS, WPR>(wr, c, lane);
      if (col < n) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (gy[c][j] - s1 - xv[c][j] * s2);
        if (dres) {
          float r[8];
          unpack8(rpk[c], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + row * lddx + col, o);
      }
    }
  }

#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = col_of<CHUNKS, WPR>(wr, c, lane);
#pragma unroll
    for (int j = 0; j < 8; ++j) { sg[col + j] = ag[c][j]; sb[col + j] = ab[c][j]; }
  }
  __syncthreads();
  for (int col = threadIdx.x; col < n; col += blockDim.x) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < RPB; ++w) {
      a += sm[(w * 2 + 0) * n_pad + col];
      b += sm[(w * 2 + 1) * n_pad + col];
    }
    partial[static_cast<long long>(blockIdx.x) * n + col] = a;
    partial[static_cast<long long>(gridDim.x + blockIdx.x) * n + col] = b;
  }
}

// out[col] (+)= sum_p partial[p][col].  Eight row groups per CTA each sum every eighth partial, then the
// groups are folded in index order: parallel enough to hide latency, and the order is fixed.
__global__ void __launch_bounds__(256)
norm_bwd_reduce_kernel(const float* __restrict__ partial, int num_partials, int n, float* __restrict__ dgamma,
                       float* __restrict__ dbeta, int accumulate) {
  __shared__ float sa[8][33], sb[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + tx;
  float a = 0.f, b = 0.f;
  if (col < n) {
    // eight independent loads per array are requested before they are added (in the same order as a plain loop):
    // the fold is a chain of dependent additions, but its loads need not wait for one another
    int p = ty;
    for (; p + 56 < num_partials; p += 64) {
      float va[8], vb[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        va[u] = partial[static_cast<long long>(p + 8 * u) * n + col];
        vb[u] = dbeta ? partial[static_cast<long long>(num_partials + p + 8 * u) * n + col] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) { a += va[u]; b += vb[u]; }
    }
    for (; p < num_partials; p += 8) {
      a += partial[static_cast<long long>(p) * n + col];
      if (dbeta) b += partial[static_cast<long long>(num_partials + p) * n + col];
    }
  }
  sa[ty][tx] = a;
  sb[ty][tx] = b;
  __syncthreads();
  if (ty == 0 && col < n) {
    float ta = 0.f, tb = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) { ta += sa[g][tx]; tb += sb[g][tx]; }
    dgamma[col] = accumulate ? dgamma[col] + ta : ta;
    if (dbeta) dbeta[col] = accumulate ? dbeta[col] + tb : tb;
  }
}

}  // namespace rb

namespace {
struct NormCfg { int chunks, wpr; };
inline NormCfg cfg_for(int n) {
  if (n <= 768) return {3, 1};        // 768-wide rows (d_model of the headline model): no idle lanes, fewer registers
  if (n <= 1024) return {4, 1};
  if (n <= 2048) return {4, 2};
  if (n <= 4096) return {4, 4};
  if (n <= 8192) return {8, 4};
  return {0, 0};
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline int rows_per_block(int n) { return rb::kNormWarps / cfg_for(n).wpr; }
}  // namespace

RB_API int rb_norm_bwd_num_partials(int rows, int n) {
  const NormCfg c = cfg_for(n);
  if (c.chunks == 0) return 0;
  const int rpb = rb::kNormWarps / c.wpr;
  const int sms = rbhost::device_sm_count();
  const int blocks_needed = (rows + rpb - 1) / rpb;
  const int grid = blocks_needed < 2 * sms ? blocks_needed : 2 * sms;
  return grid < 1 ? 1 : grid;
}

#define RB_NORM_DISPATCH(N_, MACRO)                   \
  {                                                   \
    if ((N_) <= 768) { MACRO(3, 1) }                  \
    else if ((N_) <= 1024) { MACRO(4, 1) }            \
    else if ((N_) <= 2048) { MACRO(4, 2) }            \
    else if ((N_) <= 4096) { MACRO(4, 4) }            \
    else { MACRO(8, 4) }                              \
  }

RB_API int rb_norm_fwd(const void* x, long long ldx, const void* gamma, const void* beta, void* y, long long ldy,
                       float* mean, float* rstd, int rows, int n, float eps, int rms, void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const NormCfg cfg = cfg_for(n);
  if (cfg.chunks == 0 || (n & 7) || (ldx & 7) || (ldy & 7) || rows <= 0) return -1;
  if (!aligned16(x) || !aligned16(y) || !aligned16(gamma) || (beta && !aligned16(beta))) return -2;
  const int sms = rbhost::device_sm_count();
  const int rpb = rows_per_block(n);
  const int blocks_needed = (rows + rpb - 1) / rpb;
  const int grid = blocks_needed < 8 * sms ? blocks_needed : 8 * sms;
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto G = reinterpret_cast<const __nv_bfloat16*>(gamma);
  auto B = reinterpret_cast<const __nv_bfloat16*>(beta);
  auto Y = reinterpret_cast<__nv_bfloat16*>(y);
#define RB_LAUNCH(C, W)                                                                                           \
  if (rms) rb::norm_fwd_kernel<C, W, true><<<grid, rb::kNormWarps * 32, 0, stream>>>(X, ldx, G, nullptr, Y, ldy,  \
                                                                                     nullptr, rstd, rows, n, eps);\
  else rb::norm_fwd_kernel<C, W, false><<<grid, rb::kNormWarps * 32, 0, stream>>>(X, ldx, G, B, Y, ldy, mean,     \
                                                                                  rstd, rows, n, eps);
  RB_NORM_DISPATCH(n, RB_LAUNCH)
#undef RB_LAUNCH
  return static_cast<int>(cudaGetLastError());
}

// `partial` is caller-provided scratch of 2 * rb_norm_bwd_num_partials(rows, n) * n floats.
RB_API int rb_norm_bwd(const void* dy, long long lddy, const void* x, long long ldx, const void* gamma,
                       const float* mean, const float* rstd, const void* dres, long long lddres, void* dx,
                       long long lddx, float* dgamma, float* dbeta, float* partial, int rows, int n, int rms,
                       int accumulate, void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const NormCfg cfg = cfg_for(n);
  if (cfg.chunks == 0 || (n & 7) || (ldx & 7) || (lddy & 7) || (lddx & 7) || rows <= 0) return -1;
  if (!aligned16(x) || !aligned16(dy) || !aligned16(dx) || !aligned16(gamma) || (dres && (!aligned16(dres) || (lddres & 7))))
    return -2;
  if (!partial || !dgamma || !rstd || (!rms && (!mean || !dbeta))) return -3;
  const int grid = rb_norm_bwd_num_partials(rows, n);
  const int rpb = rows_per_block(n);
  const int smem = rpb * 2 * cfg.wpr * cfg.chunks * 256 * static_cast<int>(sizeof(float));
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto G = reinterpret_cast<const __nv_bfloat16*>(gamma);
  auto DR = reinterpret_cast<const __nv_bfloat16*>(dres);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
#define RB_LAUNCH(C, W)                                                                                            \
  {                                                                                                                \
    if (rms) {                                                                                                     \
      auto k = rb::norm_bwd_kernel<C, W, true>;                                                                    \
      if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);            \
      k<<<grid, rb::kNormWarps * 32, smem, stream>>>(DY, lddy, X, ldx, G, mean, rstd, DR, lddres, DX, lddx,        \
                                                     partial, rows, n);                                            \
    } else {                                                                                                       \
      auto k = rb::norm_bwd_kernel<C, W, false>;                                                                   \
      if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);            \
      k<<<grid, rb::kNormWarps * 32, smem, stream>>>(DY, lddy, X, ldx, G, mean, rstd, DR, lddres, DX, lddx,        \
                                                     partial, rows, n);                                            \
    }                                                                                                              \
  }
  RB_NORM_DISPATCH(n, RB_LAUNCH)
#undef RB_LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  rb::norm_bwd_reduce_kernel<<<(n + 31) / 32, 256, 0, stream>>>(partial, grid, n, dgamma, rms ? nullptr : dbeta,
                                                                 accumulate);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------------------
// rb_norm_bwd_noalloc: the backward pass with its partial-sum scratch in a library-owned device array.
// ---------------------------------------------------------------------------------------------------------------
// Capacity of the built-in scratch: 2 x 296 partial rows of up to 4096 columns (9.25 MiB of fp32).  The array is
// part of the library image, so every GPU that loads this library holds it until the process exits.
constexpr long long kNoAllocScratchFloats = 2LL * 296 * 4096;
static __device__ __align__(256) float g_norm_bwd_scratch[kNoAllocScratchFloats];

RB_API long long rb_norm_bwd_noalloc_capacity_floats(void) { return kNoAllocScratchFloats; }

RB_API int rb_norm_bwd_noalloc(const void* dy, long long lddy, const void* x, long long ldx, const void* gamma,
                               const float* mean, const float* rstd, const void* dres, long long lddres, void* dx,
                               long long lddx, float* dgamma, float* dbeta, int rows, int n, int rms, int accumulate,
                               void* stream_v) {
  // In host code the array's name is only a stand-in for the device symbol; the address a kernel can use has to be
  // asked for, once per device and with that device current.
  static float* scratch_by_device[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -20;
  if (scratch_by_device[dev] == nullptr) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_norm_bwd_scratch);
    if (e != cudaSuccess || p == nullptr) return e != cudaSuccess ? static_cast<int>(e) : -21;
    scratch_by_device[dev] = p;
  }
  const int parts = rb_norm_bwd_num_partials(rows, n);
  if (parts <= 0) return -1;                                                       // unsupported row length
  if (2LL * parts * n > kNoAllocScratchFloats) return -22;                         // beyond the built-in scratch
  // The partial rows are fully overwritten by the first kernel before the second one reads them, so nothing
  // of an earlier call's contents needs clearing.
  return rb_norm_bwd(dy, lddy, x, ldx, gamma, mean, rstd, dres, lddres, dx, lddx, dgamma, dbeta, scratch_by_device[dev],
                     rows, n, rms, accumulate, stream_v);
}
