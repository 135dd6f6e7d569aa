// Elementwise, reduction and data-movement kernels: the sm_100a restatement of the reference's
// WGSL compute entry points (crates/wgpu-backend/src/shaders.wgsl: binary :14-190, unary :193-440,
// scalar :445-550, sum_reduce_full :1149, transpose_tiled :874, gather/scatter :924-996,
// broadcast_to :1029, strided_copy :1202, dropout :1238-1281, apply_mask :1294) and of the CPU
// backend's gelu / sum_dim0 / add_row_vector (crates/ndarray-backend/src/lib.rs:565,1084,318).
// One templated grid-stride kernel per family; 128-bit accesses when the pointers allow it.
#include "elementwise.h"

#include "rb_common.cuh"

namespace rb {

template <typename T> struct Cvt;
template <> struct Cvt<float> {
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
};
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
};

__device__ __forceinline__ float binary_apply(int op, float a, float b) {
  switch (op) {
    case RB_ADD: return a + b;
    case RB_MUL: return a * b;
    case RB_SUB: return a - b;
    case RB_DIV: return a / b;
    default: return fmaxf(a, b);
  }
}
__device__ __forceinline__ float unary_apply(int op, float a) {
  switch (op) {
    case RB_RELU: return fmaxf(a, 0.f);
    case RB_SIGMOID: return 1.f / (1.f + expf(-a));
    case RB_TANH: return tanhf(a);
    case RB_EXP: return expf(a);
    case RB_LOG: return logf(a);
    case RB_SQRT: return sqrtf(a);
    case RB_NEG: return -a;
    case RB_GELU: return gelu_tanh(a);
    case RB_SILU: return silu(a);
    default: return a;
  }
}
__device__ __forceinline__ float unary_grad(int op, float x) {
  switch (op) {
    case RB_RELU: return x > 0.f ? 1.f : 0.f;
    case RB_SIGMOID: { const float s = 1.f / (1.f + expf(-x)); return s * (1.f - s); }
    case RB_TANH: { const float t = tanhf(x); return 1.f - t * t; }
    case RB_GELU: return gelu_tanh_grad(x);
    case RB_SILU: return silu_grad(x);
    default: return 1.f;
  }
}
__device__ __forceinline__ float scalar_apply(int op, float a, float s) {
  switch (op) {
    case RB_ADD_SCALAR: return a + s;
    case RB_MUL_SCALAR: return a * s;
    case RB_GT_SCALAR: return a > s ? 1.f : 0.f;
    default: return s;
  }
}

// MODE 0 binary, 1 unary, 2 scalar, 3 unary backward (b = dy), 4 mask (b = mask)
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
pointwise_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, float s, T* __restrict__ out, long long n) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float x = (MODE == 2 && op == RB_FILL) ? 0.f : Cvt<T>::ld(a + i);
    float r;
    if (MODE == 0) r = binary_apply(op, x, Cvt<T>::ld(b + i));
    else if (MODE == 1) r = unary_apply(op, x);
    else if (MODE == 2) r = scalar_apply(op, x, s);
    else if (MODE == 3) r = Cvt<T>::ld(b + i) * unary_grad(op, x);
    else r = Cvt<T>::ld(b + i) > 0.f ? x : s;
    Cvt<T>::st(out + i, r);
  }
}

// 8 x bf16 / 4 x fp32 per thread per step; used when everything is 16-byte aligned.
template <int MODE>
__global__ void __launch_bounds__(256)
pointwise_bf16x8_kernel(int op, const uint4* __restrict__ a, const uint4* __restrict__ b, float s, uint4* __restrict__ out, long long n8) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    uint4 ua = (MODE == 2 && op == RB_FILL) ? make_uint4(0, 0, 0, 0) : a[i];
    uint4 ub = (MODE == 0 || MODE == 3 || MODE == 4) ? b[i] : make_uint4(0, 0, 0, 0);
    uint32_t* pa = reinterpret_cast<uint32_t*>(&ua);
    uint32_t* pb = reinterpret_cast<uint32_t*>(&ub);
    uint4 uo;
    uint32_t* po = reinterpret_cast<uint32_t*>(&uo);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = unpack_bf16x2(pa[j]);
      const float2 y = unpack_bf16x2(pb[j]);
      float r0, r1;
      if (MODE == 0) { r0 = binary_apply(op, x.x, y.x); r1 = binary_apply(op, x.y, y.y); }
      else if (MODE == 1) { r0 = unary_apply(op, x.x); r1 = unary_apply(op, x.y); }
      else if (MODE == 2) { r0 = scalar_apply(op, x.x, s); r1 = scalar_apply(op, x.y, s); }
      else if (MODE == 3) { r0 = y.x * unary_grad(op, x.x); r1 = y.y * unary_grad(op, x.y); }
      else { r0 = y.x > 0.f ? x.x : s; r1 = y.y > 0.f ? x.y : s; }
      po[j] = pack_bf16x2(r0, r1);
    }
    out[i] = uo;
  }
}

inline int ew_grid(long long n) {
  long long blocks = (n + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

template <int MODE>
int launch_pointwise(int op, const void* a, const void* b, float s, void* out, long long n, int dtype, cudaStream_t st) {
  if (n <= 0) return 0;
  if (dtype == 1) {
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out);
    const long long n8 = ((bits & 15) == 0) ? n / 8 : 0;
    if (n8 > 0)
      pointwise_bf16x8_kernel<MODE><<<ew_grid(n8), 256, 0, st>>>(op, reinterpret_cast<const uint4*>(a),
                                                                 reinterpret_cast<const uint4*>(b), s,
                                                                 reinterpret_cast<uint4*>(out), n8);
    const long long done = n8 * 8;
    if (done < n) {
      auto A = reinterpret_cast<const __nv_bfloat16*>(a);
      auto B = reinterpret_cast<const __nv_bfloat16*>(b);
      pointwise_kernel<__nv_bfloat16, MODE><<<ew_grid(n - done), 256, 0, st>>>(
          op, A ? A + done : A, B ? B + done : B, s, reinterpret_cast<__nv_bfloat16*>(out) + done, n - done);
    }
  } else {
    pointwise_kernel<float, MODE><<<ew_grid(n), 256, 0, st>>>(op, reinterpret_cast<const float*>(a),
                                                              reinterpret_cast<const float*>(b), s,
                                                              reinterpret_cast<float*>(out), n);
  }
  return static_cast<int>(cudaGetLastError());
}

template <typename T>
__global__ void __launch_bounds__(256)
add_row_vector_kernel(const T* __restrict__ a, const T* __restrict__ v, T* __restrict__ out, long long rows, int cols) {
  const long long n = rows * cols;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    Cvt<T>::st(out + i, Cvt<T>::ld(a + i) + Cvt<T>::ld(v + (i % cols)));
}

// Column sums in two ordered stages: stage 1 sums a slab of rows per CTA into smem partials
// (threads own columns, so accesses are coalesced), stage 2 folds the slabs.
constexpr int kSumDim0Slabs = 128;
template <typename T>
__global__ void __launch_bounds__(256)
sum_dim0_stage1(const T* __restrict__ a, long long lda, float* __restrict__ partial, long long rows, int cols) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  const int slab = blockIdx.y;
  const long long per = (rows + gridDim.y - 1) / gridDim.y;
  const long long lo = per * slab;
  const long long hi = lo + per < rows ? lo + per : rows;
  if (col >= cols) return;
  float acc = 0.f;
  for (long long r = lo; r < hi; ++r) acc += Cvt<T>::ld(a + r * lda + col);
  partial[static_cast<long long>(slab) * cols + col] = acc;
}
// bf16 fast path of stage 1: a thread owns 8 adjacent columns (one 16-byte load per row) and every 8th row of the
// slab; the 8 row lanes of a column group are folded through shared memory in lane order (deterministic).
__global__ void __launch_bounds__(256)
sum_dim0_stage1_vec(const __nv_bfloat16* __restrict__ a, long long lda, float* __restrict__ partial, long long rows, int cols) {
  __shared__ float sh[8][32][9];
  const int cg = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + cg) * 8;
  const int slab = blockIdx.y;
  const long long per = (rows + gridDim.y - 1) / gridDim.y;
  const long long lo = per * slab;
  const long long hi = lo + per < rows ? lo + per : rows;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < cols) {
    long long r = lo + ry;
    for (; r + 56 < hi; r += 64) {                       // eight independent 16-byte loads in flight
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldg(reinterpret_cast<const uint4*>(a + (r + 8 * u) * lda + col));
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&v[u]);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(w[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
      }
    }
    for (; r < hi; r += 8) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(a + r * lda + col));
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(w[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sh[ry][cg][j] = acc[j];
  __syncthreads();
  // 256 threads fold 256 columns: thread t owns column (t / 8 group, t % 8)
  const int g2 = threadIdx.x >> 3, j2 = threadIdx.x & 7;
  const int c2 = (blockIdx.x * 32 + g2) * 8 + j2;
  if (c2 < cols) {
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 8; ++y) t += sh[y][g2][j2];
    partial[static_cast<long long>(slab) * cols + c2] = t;
  }
}
__global__ void __launch_bounds__(256)
sum_dim0_stage2(const float* __restrict__ partial, int slabs, float* __restrict__ out, int cols, int accumulate) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= cols) return;
  float acc = 0.f;
  int s = 0;
  for (; s + 7 < slabs; s += 8) {          // the loads of eight slabs are requested together, then added in slab order
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = partial[static_cast<long long>(s + u) * cols + col];
#pragma unroll
    for (int u = 0; u < 8; ++u) acc += v[u];
  }
  for (; s < slabs; ++s) acc += partial[static_cast<long long>(s) * cols + col];
  out[col] = accumulate ? out[col] + acc : acc;
}
// Single-kernel variant for when no scratch is available: one thread per column walks all rows.
template <typename T>
__global__ void __launch_bounds__(256)
sum_dim0_direct(const T* __restrict__ a, long long lda, float* __restrict__ out, long long rows, int cols, int accumulate) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= cols) return;
  float acc = 0.f;
  for (long long r = 0; r < rows; ++r) acc += Cvt<T>::ld(a + r * lda + col);
  out[col] = accumulate ? out[col] + acc : acc;
}

template <typename T>
__global__ void __launch_bounds__(256) sum_all_stage1(const T* __restrict__ a, long long n, float* __restrict__ scratch) {
  __shared__ float sh[8];
  const long long per = (n + gridDim.x - 1) / gridDim.x;
  const long long lo = per * blockIdx.x;
  const long long hi = lo + per < n ? lo + per : n;
  float acc = 0.f;
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) acc += Cvt<T>::ld(a + i);
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += sh[w];
    scratch[blockIdx.x] = t;
  }
}
__global__ void __launch_bounds__(256) sum_all_stage2(const float* __restrict__ scratch, int nb, float* out) {
  __shared__ float sh[256];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nb; i += 256) acc += scratch[i];
  sh[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = sh[0];
}

template <typename T>
__global__ void transpose_kernel(const T* __restrict__ a, T* __restrict__ out, int rows, int cols) {
  __shared__ T tile[32][33];
  const int bx = blockIdx.x * 32, by = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = by + j, c = bx + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = a[static_cast<long long>(r) * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = bx + j, r = by + threadIdx.x;
    if (r < rows && c < cols) out[static_cast<long long>(c) * rows + r] = tile[threadIdx.x][j];
  }
}

template <typename T, bool SCATTER>
__global__ void __launch_bounds__(256)
rows_kernel(const T* __restrict__ a, const long long* __restrict__ idx, T* __restrict__ out, long long n_idx, int cols,
            long long limit RB_BOUNDS_PARAM) {
  const long long n = n_idx * cols;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long r = i / cols;
    const int c = static_cast<int>(i - r * cols);
    const long long j = idx[r];
    if (j < 0 || j >= limit) {           // out-of-range indices are skipped, never dereferenced
      if (c == 0) RB_BOUNDS_HIT(102);
      continue;
    }
    if (SCATTER) out[j * cols + c] = a[i];
    else out[i] = a[j * cols + c];
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
broadcast_kernel(const T* __restrict__ a, T* __restrict__ out, long long arows, long long acols, long long rows, long long cols) {
  const long long n = rows * cols;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long r = i / cols, c = i - r * cols;
    out[i] = a[(r % arows) * acols + (c % acols)];
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
strided_copy_kernel(const T* __restrict__ a, long long lda, T* __restrict__ out, long long ldo, long long rows, long long cols) {
  const long long n = rows * cols;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long r = i / cols, c = i - r * cols;
    out[r * ldo + c] = a[r * lda + c];
  }
}

// Philox-4x32-10
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t (&k)[2]) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k[0], n1 = lo1, n2 = hi0 ^ c[3] ^ k[1], n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
  k[0] += 0x9E3779B9u; k[1] += 0xBB67AE85u;
}
__device__ __forceinline__ void philox4(unsigned long long seed, unsigned long long ctr, uint32_t (&out)[4]) {
  uint32_t c[4] = {static_cast<uint32_t>(ctr), static_cast<uint32_t>(ctr >> 32), 0u, 0u};
  uint32_t k[2] = {static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)};
#pragma unroll
  for (int r = 0; r < 10; ++r) philox_round(c, k);
#pragma unroll
  for (int j = 0; j < 4; ++j) out[j] = c[j];
}
__device__ __forceinline__ uint32_t pcg_hash(uint32_t v) {
  const uint32_t state = v * 747796405u + 2891336453u;
  const uint32_t word = ((state >> ((state >> 28u) + 4u)) ^ state) * 277803737u;
  return (word >> 22u) ^ word;
}

template <typename T>
__global__ void __launch_bounds__(256)
dropout_kernel(const T* __restrict__ a, T* __restrict__ out, unsigned char* __restrict__ mask_out, long long n, float p,
               unsigned long long seed, unsigned long long offset, int rng) {
  const float scale = 1.f / (1.f - p);
  const long long groups = (n + 3) / 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long gi = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; gi < groups; gi += stride) {
    uint32_t r[4];
    if (rng == 0) {
      philox4(seed, offset + static_cast<unsigned long long>(gi), r);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        r[j] = pcg_hash(static_cast<uint32_t>(seed) + static_cast<uint32_t>(gi * 4 + j) * 12345u);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long i = gi * 4 + j;
      if (i < n) {
        const float u = static_cast<float>(r[j]) * (1.f / 4294967296.f);
        const bool keep = u >= p;
        Cvt<T>::st(out + i, keep ? Cvt<T>::ld(a + i) * scale : 0.f);
        if (mask_out) mask_out[i] = keep ? 1 : 0;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) argmax_rows_kernel(const T* __restrict__ a, long long lda, long long* __restrict__ out, int cols) {
  __shared__ float sv[4];
  __shared__ int si[4];
  const long long row = blockIdx.x;
  float best = -INFINITY;
  int bi = 0;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = Cvt<T>::ld(a + row * lda + c);
    if (v > best) { best = v; bi = c; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 4; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    out[row] = bi;
  }
}

}  // namespace rb

#define RB_STREAM reinterpret_cast<cudaStream_t>(stream_v)

RB_API int rb_binary(int op, const void* a, const void* b, void* out, long long n, int dtype, void* stream_v) {
  return rb::launch_pointwise<0>(op, a, b, 0.f, out, n, dtype, RB_STREAM);
}
RB_API int rb_unary(int op, const void* a, void* out, long long n, int dtype, void* stream_v) {
  return rb::launch_pointwise<1>(op, a, nullptr, 0.f, out, n, dtype, RB_STREAM);
}
RB_API int rb_scalar(int op, const void* a, float s, void* out, long long n, int dtype, void* stream_v) {
  return rb::launch_pointwise<2>(op, a, nullptr, s, out, n, dtype, RB_STREAM);
}
RB_API int rb_unary_bwd(int op, const void* x, const void* dy, void* out, long long n, int dtype, void* stream_v) {
  return rb::launch_pointwise<3>(op, x, dy, 0.f, out, n, dtype, RB_STREAM);
}
RB_API int rb_apply_mask(const void* a, const void* mask, float mask_value, void* out, long long n, int dtype, void* stream_v) {
  return rb::launch_pointwise<4>(0, a, mask, mask_value, out, n, dtype, RB_STREAM);
}

#define RB_BY_DTYPE(CALL_F32, CALL_BF16) \
  if (dtype == 0) { CALL_F32; } else { CALL_BF16; } \
  return static_cast<int>(cudaGetLastError());

RB_API int rb_add_row_vector(const void* a, const void* v, void* out, long long rows, int cols, int dtype, void* stream_v) {
  if (rows <= 0 || cols <= 0) return 0;
  const int grid = rb::ew_grid(rows * cols);
  RB_BY_DTYPE((rb::add_row_vector_kernel<float><<<grid, 256, 0, RB_STREAM>>>((const float*)a, (const float*)v, (float*)out, rows, cols)),
              (rb::add_row_vector_kernel<__nv_bfloat16><<<grid, 256, 0, RB_STREAM>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)v, (__nv_bfloat16*)out, rows, cols)))
}

RB_API int rb_sum_dim0(const void* a, long long lda, float* out, long long rows, int cols, int dtype, int accumulate, void* stream_v) {
  if (rows <= 0 || cols <= 0) return 0;
  const int grid = (cols + 255) / 256;
  RB_BY_DTYPE((rb::sum_dim0_direct<float><<<grid, 256, 0, RB_STREAM>>>((const float*)a, lda, out, rows, cols, accumulate)),
              (rb::sum_dim0_direct<__nv_bfloat16><<<grid, 256, 0, RB_STREAM>>>((const __nv_bfloat16*)a, lda, out, rows, cols, accumulate)))
}

// Scratch-backed two-stage column sum: partial must hold rb_sum_dim0_slabs() * cols floats.
RB_API int rb_sum_dim0_slabs(void) { return rb::kSumDim0Slabs; }
RB_API int rb_sum_dim0_staged(const void* a, long long lda, float* out, float* partial, long long rows, int cols, int dtype,
                              int accumulate, void* stream_v) {
  if (rows <= 0 || cols <= 0) return 0;
  if (!partial) return -1;
  int slabs = rb::kSumDim0Slabs;
  if (rows < slabs) slabs = static_cast<int>(rows);
  dim3 grid((cols + 255) / 256, slabs);
  if (dtype == 0) rb::sum_dim0_stage1<float><<<grid, 256, 0, RB_STREAM>>>((const float*)a, lda, partial, rows, cols);
  else if ((cols % 8 == 0) && (lda % 8 == 0) && (reinterpret_cast<uintptr_t>(a) % 16 == 0))
    rb::sum_dim0_stage1_vec<<<dim3((cols + 255) / 256, slabs), 256, 0, RB_STREAM>>>((const __nv_bfloat16*)a, lda, partial, rows, cols);
  else rb::sum_dim0_stage1<__nv_bfloat16><<<grid, 256, 0, RB_STREAM>>>((const __nv_bfloat16*)a, lda, partial, rows, cols);
  rb::sum_dim0_stage2<<<(cols + 255) / 256, 256, 0, RB_STREAM>>>(partial, slabs, out, cols, accumulate);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_sum_all(const void* a, long long n, int dtype, float* scratch, float* out, void* stream_v) {
  if (n <= 0 || !scratch || !out) return -1;
  long long want = (n + 4095) / 4096;
  const int nb = static_cast<int>(want < 1024 ? (want < 1 ? 1 : want) : 1024);
  if (dtype == 0) rb::sum_all_stage1<float><<<nb, 256, 0, RB_STREAM>>>((const float*)a, n, scratch);
  else rb::sum_all_stage1<__nv_bfloat16><<<nb, 256, 0, RB_STREAM>>>((const __nv_bfloat16*)a, n, scratch);
  rb::sum_all_stage2<<<1, 256, 0, RB_STREAM>>>(scratch, nb, out);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_transpose(const void* a, void* out, int rows, int cols, int dtype, void* stream_v) {
  if (rows <= 0 || cols <= 0) return 0;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  RB_BY_DTYPE((rb::transpose_kernel<float><<<grid, block, 0, RB_STREAM>>>((const float*)a, (float*)out, rows, cols)),
              (rb::transpose_kernel<__nv_bfloat16><<<grid, block, 0, RB_STREAM>>>((const __nv_bfloat16*)a, (__nv_bfloat16*)out, rows, cols)))
}

RB_API int rb_gather_rows(const void* a, const long long* idx, void* out, long long n_idx, int cols, long long src_rows, int dtype, void* stream_v) {
  if (n_idx <= 0 || cols <= 0) return 0;
  const int grid = rb::ew_grid(n_idx * cols);
  RB_BY_DTYPE((rb::rows_kernel<float, false><<<grid, 256, 0, RB_STREAM>>>((const float*)a, idx, (float*)out, n_idx, cols, src_rows RB_BOUNDS_ARG)),
              (rb::rows_kernel<__nv_bfloat16, false><<<grid, 256, 0, RB_STREAM>>>((const __nv_bfloat16*)a, idx, (__nv_bfloat16*)out, n_idx, cols, src_rows RB_BOUNDS_ARG)))
}
RB_API int rb_scatter_rows(const void* a, const long long* idx, void* out, long long n_idx, int cols, long long dst_rows, int dtype, void* stream_v) {
  if (n_idx <= 0 || cols <= 0) return 0;
  const int grid = rb::ew_grid(n_idx * cols);
  RB_BY_DTYPE((rb::rows_kernel<float, true><<<grid, 256, 0, RB_STREAM>>>((const float*)a, idx, (float*)out, n_idx, cols, dst_rows RB_BOUNDS_ARG)),
              (rb::rows_kernel<__nv_bfloat16, true><<<grid, 256, 0, RB_STREAM>>>((const __nv_bfloat16*)a, idx, (__nv_bfloat16*)out, n_idx, cols, dst_rows RB_BOUNDS_ARG)))
}
RB_API int rb_broadcast_to(const void* a, void* out, long long arows, long long acols, long long rows, long long cols, int dtype, void* stream_v) {
  if (rows <= 0 || cols <= 0 || arows <= 0 || acols <= 0) return -1;
  const int grid = rb::ew_grid(rows * cols);
  RB_BY_DTYPE((rb::broadcast_kernel<float><<<grid, 256, 0, RB_STREAM>>>((const float*)a, (float*)out, arows, acols, rows, cols)),
              (rb::broadcast_kernel<__nv_bfloat16><<<grid, 256, 0, RB_STREAM>>>((const __nv_bfloat16*)a, (__nv_bfloat16*)out, arows, acols, rows, cols)))
}
RB_API int rb_strided_copy(const void* a, long long lda, void* out, long long ldo, long long rows, long long cols, int dtype, void* stream_v) {
  if (rows <= 0 || cols <= 0) return 0;
  const int grid = rb::ew_grid(rows * cols);
  RB_BY_DTYPE((rb::strided_copy_kernel<float><<<grid, 256, 0, RB_STREAM>>>((const float*)a, lda, (float*)out, ldo, rows, cols)),
              (rb::strided_copy_kernel<__nv_bfloat16><<<grid, 256, 0, RB_STREAM>>>((const __nv_bfloat16*)a, lda, (__nv_bfloat16*)out, ldo, rows, cols)))
}
RB_API int rb_dropout(const void* a, void* out, unsigned char* mask_out, long long n, float p, unsigned long long seed,
                      unsigned long long offset, int rng, int dtype, void* stream_v) {
  if (n <= 0) return 0;
  if (p < 0.f || p >= 1.f) return -1;
  const int grid = rb::ew_grid((n + 3) / 4);
  RB_BY_DTYPE((rb::dropout_kernel<float><<<grid, 256, 0, RB_STREAM>>>((const float*)a, (float*)out, mask_out, n, p, seed, offset, rng)),
              (rb::dropout_kernel<__nv_bfloat16><<<grid, 256, 0, RB_STREAM>>>((const __nv_bfloat16*)a, (__nv_bfloat16*)out, mask_out, n, p, seed, offset, rng)))
}
RB_API int rb_argmax_rows(const void* a, long long lda, long long* out, long long rows, int cols, int dtype, void* stream_v) {
  if (rows <= 0 || cols <= 0) return 0;
  RB_BY_DTYPE((rb::argmax_rows_kernel<float><<<static_cast<int>(rows), 128, 0, RB_STREAM>>>((const float*)a, lda, out, cols)),
              (rb::argmax_rows_kernel<__nv_bfloat16><<<static_cast<int>(rows), 128, 0, RB_STREAM>>>((const __nv_bfloat16*)a, lda, out, cols)))
}
