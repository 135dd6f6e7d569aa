// Fused optimizer kernels over flat fp32 state: Adam / AdamW with optional global-norm clipping and
// overflow skip decided on the device, SGD with momentum, the ordered sum-of-squares reduction the
// clipping needs, and the fp32 <-> bf16 casts.
//
// One pass over (p, m, v, g) replaces the reference's ~14 tensor ops and ~8 full-size constant
// tensors per parameter per step (crates/optim/src/lib.rs:433-514).  Weight decay is decoupled when
// `decoupled` is set, which is what "AdamW" means; the reference's alias folds it into the gradient
// (crates/optim/src/lib.rs:464-470,604) and that behaviour is available with decoupled = 0.
#include "optim.h"

#include "rb_common.cuh"

namespace rb {

template <bool G_BF16>
__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, const void* __restrict__ g_v,
            __nv_bfloat16* __restrict__ p_bf16, long long n, RbAdamArgs a, const float* __restrict__ grad_norm,
            const int* __restrict__ found_inf) {
  if (found_inf != nullptr && *found_inf != 0) return;   // overflow: skip the whole step
  float gscale = a.grad_scale;
  if (a.max_grad_norm > 0.f && grad_norm != nullptr) {
    const float gn = *grad_norm;
    const float coef = a.max_grad_norm / (gn + 1e-6f);
    if (coef < 1.f) gscale *= coef;
  }
  const float inv_bc1 = 1.f / a.bias_correction1;
  const float inv_bc2 = 1.f / a.bias_correction2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 pp = *reinterpret_cast<float4*>(p + i);
      float4 mm = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      float gg[4];
      if (G_BF16) {
        uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(g_v) + i);
        float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y);
        gg[0] = a0.x; gg[1] = a0.y; gg[2] = a1.x; gg[3] = a1.y;
      } else {
        float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g_v) + i);
        gg[0] = t.x; gg[1] = t.y; gg[2] = t.z; gg[3] = t.w;
      }
      float pa[4] = {pp.x, pp.y, pp.z, pp.w}, ma[4] = {mm.x, mm.y, mm.z, mm.w}, va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float g = gg[j] * gscale;
        if (!a.decoupled) g += a.weight_decay * pa[j];
        ma[j] = a.beta1 * ma[j] + (1.f - a.beta1) * g;
        va[j] = a.beta2 * va[j] + (1.f - a.beta2) * g * g;
        const float mhat = ma[j] * inv_bc1;
        const float vhat = va[j] * inv_bc2;
        float upd = mhat / (sqrtf(vhat) + a.eps);
        if (a.decoupled) upd += a.weight_decay * pa[j];
        pa[j] -= a.lr * upd;
      }
      *reinterpret_cast<float4*>(p + i) = make_float4(pa[0], pa[1], pa[2], pa[3]);
      *reinterpret_cast<float4*>(m + i) = make_float4(ma[0], ma[1], ma[2], ma[3]);
      *reinterpret_cast<float4*>(v + i) = make_float4(va[0], va[1], va[2], va[3]);
      if (p_bf16) {
        uint2 o;
        o.x = pack_bf16x2(pa[0], pa[1]);
        o.y = pack_bf16x2(pa[2], pa[3]);
        *reinterpret_cast<uint2*>(p_bf16 + i) = o;
      }
    } else {
      for (long long k = i; k < n; ++k) {
        float g = (G_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g_v)[k])
                          : reinterpret_cast<const float*>(g_v)[k]) * gscale;
        float pk = p[k];
        if (!a.decoupled) g += a.weight_decay * pk;
        const float mk = a.beta1 * m[k] + (1.f - a.beta1) * g;
        const float vk = a.beta2 * v[k] + (1.f - a.beta2) * g * g;
        float upd = (mk * inv_bc1) / (sqrtf(vk * inv_bc2) + a.eps);
        if (a.decoupled) upd += a.weight_decay * pk;
        pk -= a.lr * upd;
        p[k] = pk; m[k] = mk; v[k] = vk;
        if (p_bf16) p_bf16[k] = __float2bfloat16(pk);
      }
    }
  }
}

template <bool G_BF16>
__global__ void __launch_bounds__(256)
sgd_kernel(float* __restrict__ p, float* __restrict__ mom, const void* __restrict__ g_v,
           __nv_bfloat16* __restrict__ p_bf16, long long n, float lr, float momentum, float wd, float gscale) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float g = (G_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g_v)[i])
                      : reinterpret_cast<const float*>(g_v)[i]) * gscale;
    float pk = p[i];
    g += wd * pk;
    if (mom != nullptr && momentum != 0.f) {
      const float b = momentum * mom[i] + g;
      mom[i] = b;
      g = b;
    }
    pk -= lr * g;
    p[i] = pk;
    if (p_bf16) p_bf16[i] = __float2bfloat16(pk);
  }
}

constexpr int kSumsqBlocks = 1024;

template <bool BF16>
__global__ void __launch_bounds__(256)
sumsq_stage1(const void* __restrict__ x_v, long long n, float* __restrict__ scratch, int* __restrict__ found_inf) {
  __shared__ float sh[8];
  float acc = 0.f;
  bool bad = false;
  // contiguous slab per block, fixed order inside: reproducible
  const long long per_block = (n + gridDim.x - 1) / gridDim.x;
  const long long lo = per_block * blockIdx.x;
  const long long hi = lo + per_block < n ? lo + per_block : n;
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x_v)[i])
                         : reinterpret_cast<const float*>(x_v)[i];
    if (!isfinite(v)) bad = true;
    acc += v * v;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  if (bad && found_inf) *found_inf = 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += sh[w];
    scratch[blockIdx.x] = t;
  }
}
__global__ void __launch_bounds__(256) sumsq_stage2(const float* __restrict__ scratch, int nblocks, float* out, int accumulate) {
  __shared__ float sh[256];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nblocks; i += 256) acc += scratch[i];
  sh[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + sh[0] : sh[0];
}
__global__ void sqrt_scalar_kernel(const float* in, float* out) { out[0] = sqrtf(in[0]); }

__global__ void __launch_bounds__(256) cast_f32_bf16_kernel(const float* __restrict__ s, __nv_bfloat16* __restrict__ d, long long n) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 t = *reinterpret_cast<const float4*>(s + i);
      uint2 o;
      o.x = pack_bf16x2(t.x, t.y);
      o.y = pack_bf16x2(t.z, t.w);
      *reinterpret_cast<uint2*>(d + i) = o;
    } else {
      for (long long k = i; k < n; ++k) d[k] = __float2bfloat16(s[k]);
    }
  }
}
__global__ void __launch_bounds__(256) cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ s, float* __restrict__ d, long long n) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    d[i] = __bfloat162float(s[i]);
}

inline int grid_for(long long n, int per_thread) {
  long long blocks = (n + 256LL * per_thread - 1) / (256LL * per_thread);
  const long long cap = 148LL * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace rb

RB_API int rb_adam_step(float* p, float* m, float* v, const void* g, int g_bf16, void* p_bf16, long long n,
                        const RbAdamArgs* args, const float* grad_norm, const int* found_inf, void* stream_v) {
  if (n <= 0) return 0;
  if (!p || !m || !v || !g || !args) return -1;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(g)) & 15)
    return -2;
  if (p_bf16 && (reinterpret_cast<uintptr_t>(p_bf16) & 7)) return -2;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const int grid = rb::grid_for(n, 4);
  if (g_bf16)
    rb::adam_kernel<true><<<grid, 256, 0, stream>>>(p, m, v, g, reinterpret_cast<__nv_bfloat16*>(p_bf16), n, *args,
                                                    grad_norm, found_inf);
  else
    rb::adam_kernel<false><<<grid, 256, 0, stream>>>(p, m, v, g, reinterpret_cast<__nv_bfloat16*>(p_bf16), n, *args,
                                                     grad_norm, found_inf);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_sgd_step(float* p, float* mom, const void* g, int g_bf16, void* p_bf16, long long n, float lr,
                       float momentum, float weight_decay, float grad_scale, void* stream_v) {
  if (n <= 0) return 0;
  if (!p || !g) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const int grid = rb::grid_for(n, 1);
  if (g_bf16)
    rb::sgd_kernel<true><<<grid, 256, 0, stream>>>(p, mom, g, reinterpret_cast<__nv_bfloat16*>(p_bf16), n, lr,
                                                   momentum, weight_decay, grad_scale);
  else
    rb::sgd_kernel<false><<<grid, 256, 0, stream>>>(p, mom, g, reinterpret_cast<__nv_bfloat16*>(p_bf16), n, lr,
                                                    momentum, weight_decay, grad_scale);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_sumsq_scratch_floats(void) { return rb::kSumsqBlocks; }

RB_API int rb_sumsq(const void* x, int is_bf16, long long n, float* scratch, float* out, int* found_inf,
                    int accumulate, void* stream_v) {
  if (n <= 0 || !x || !scratch || !out) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  long long want = (n + 4095) / 4096;
  const int blocks = static_cast<int>(want < rb::kSumsqBlocks ? (want < 1 ? 1 : want) : rb::kSumsqBlocks);
  if (is_bf16) rb::sumsq_stage1<true><<<blocks, 256, 0, stream>>>(x, n, scratch, found_inf);
  else rb::sumsq_stage1<false><<<blocks, 256, 0, stream>>>(x, n, scratch, found_inf);
  rb::sumsq_stage2<<<1, 256, 0, stream>>>(scratch, blocks, out, accumulate);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_sqrt_scalar(const float* in, float* out, void* stream_v) {
  rb::sqrt_scalar_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(in, out);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream_v) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 7)) return -2;
  rb::cast_f32_bf16_kernel<<<rb::grid_for(n, 4), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      src, reinterpret_cast<__nv_bfloat16*>(dst), n);
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_cast_bf16_to_f32(const void* src, float* dst, long long n, void* stream_v) {
  if (n <= 0) return 0;
  rb::cast_bf16_f32_kernel<<<rb::grid_for(n, 1), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), dst, n);
  return static_cast<int>(cudaGetLastError());
}
