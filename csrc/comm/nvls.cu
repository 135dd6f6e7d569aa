// In-switch reductions and broadcasts over NVLink multicast (NVLS): `multimem.ld_reduce` sums one address over every
// GPU bound to a multicast object inside the NVSwitch and returns the total, `multimem.st` writes one value to all of
// them.  The buffers come from torch.distributed's symmetric memory (it creates the multicast object and binds every
// rank's allocation; `rustral_b200/parallel/nvls.py`), the kernels here are the data plane:
//
//   rb_mc_reduce_f32      dst[i] (+)= sum over ranks of buf_r[offset + i]          (reduce-scatter of one rank's slice)
//   rb_mc_allreduce       in place over the whole buffer: every rank reduces its 1 / world slice through the switch and
//                         multimem-stores the result to all ranks (fp32 or bf16 elements, fp32 accumulation)
//   rb_mc_broadcast       multimem.st of a local source range into everybody's buffer (parameter push)
//
// Ordering between ranks is the caller's: the flag kernels of symm.cu / zero3.cu (bounded waits) bracket these calls.
// A replacement of the NCCL calls the reference only stubs (crates/distributed/src/nccl.rs:240-262,283-346).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "flags.cuh"
#include "nvls.h"
#include "rb_common.cuh"

namespace rb {

__device__ __forceinline__ float4 mc_ld_reduce_f32x4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_f32x4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// eight bf16 values: the switch accumulates in fp32 (.acc::f32) and returns bf16 pairs
__device__ __forceinline__ uint4 mc_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_b32x4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// four reductions in flight per thread: a multimem.ld_reduce is a round trip to the switch
__global__ void __launch_bounds__(256)
mc_reduce_f32_kernel(const float* __restrict__ mc, float* __restrict__ dst, long long n4, int accumulate) {
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * step < n4; i += 4 * step) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = mc_ld_reduce_f32x4(mc + 4 * (i + u * step));
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float4* d = reinterpret_cast<float4*>(dst) + i + u * step;
      if (accumulate) {
        const float4 o = *d;
        v[u].x += o.x; v[u].y += o.y; v[u].z += o.z; v[u].w += o.w;
      }
      *d = v[u];
    }
  }
  for (; i < n4; i += step) {
    float4 v = mc_ld_reduce_f32x4(mc + 4 * i);
    float4* d = reinterpret_cast<float4*>(dst) + i;
    if (accumulate) {
      const float4 o = *d;
      v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
    }
    *d = v;
  }
}

// 16-byte units [first, first + count) of the buffer: reduce through the switch, store back to every rank
template <bool BF16>
__global__ void __launch_bounds__(256)
mc_allreduce_kernel(void* mc, long long first, long long count) {
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  uint4* base = reinterpret_cast<uint4*>(mc) + first;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += step) {
    if (BF16) {
      mc_st_b32x4(base + i, mc_ld_reduce_bf16x8(base + i));
    } else {
      mc_st_f32x4(reinterpret_cast<float*>(base + i), mc_ld_reduce_f32x4(reinterpret_cast<const float*>(base + i)));
    }
  }
}

__global__ void __launch_bounds__(256)
mc_broadcast_kernel(const uint4* __restrict__ src, void* mc, long long count) {
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  uint4* base = reinterpret_cast<uint4*>(mc);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += step)
    mc_st_b32x4(base + i, __ldg(src + i));
}

// One-shot all-reduce of a small activation for tensor-parallel inference: raise this rank's flag on every peer, wait
// (bounded) for all flags, then every rank reads the whole tensor through the multicast address, i.e. summed inside the
// switch (bf16 pairs, fp32 accumulation), adds the residual and writes its own output.  One load per 16 bytes instead of
// one per rank, and `world` times fewer bytes into each GPU than the peer-load kernel (`rb_tp_allreduce`).
__global__ void __launch_bounds__(256)
tp_allreduce_mc_kernel(const void* __restrict__ mc_stage, void* const* __restrict__ pad_ptrs, const unsigned int* __restrict__ local_pad,
                       int world, int rank, int channel, const unsigned int* __restrict__ epoch_dev, unsigned long long limit_ns,
                       const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out, long long n8,
                       unsigned int* status) {
  __shared__ int ok_s;
  const unsigned int epoch = *epoch_dev;
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned int*>(pad_ptrs[threadIdx.x]) + channel * world + rank, epoch);
  }
  if (threadIdx.x == 0) ok_s = wait_flags(local_pad, world, channel, epoch, limit_ns, status, 130 + channel) ? 1 : 0;
  __syncthreads();
  if (!ok_s) return;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    uint4 u = mc_ld_reduce_bf16x8(reinterpret_cast<const uint4*>(mc_stage) + i);
    if (residual) {
      const uint4 r = __ldg(reinterpret_cast<const uint4*>(residual) + i);
      const uint32_t* pu = reinterpret_cast<const uint32_t*>(&u);
      const uint32_t* pr = reinterpret_cast<const uint32_t*>(&r);
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = unpack_bf16x2(pu[j]), b = unpack_bf16x2(pr[j]);
        o[j] = pack_bf16x2(a.x + b.x, a.y + b.y);
      }
      u = make_uint4(o[0], o[1], o[2], o[3]);
    }
    reinterpret_cast<uint4*>(out)[i] = u;
  }
}

}  // namespace rb

namespace {
inline int mc_grid(long long units, int max_ctas) {
  long long b = (units + 255) / 256;
  const long long cap = max_ctas > 0 ? max_ctas : 148 * 4;
  if (b > cap) b = cap;
  return static_cast<int>(b > 0 ? b : 1);
}
}  // namespace

RB_API int rb_mc_reduce_f32(const void* mc, long long elem_offset, void* dst, long long n, int accumulate, int max_ctas, void* stream) {
  if (!mc || !dst || n <= 0 || (n & 3) || (elem_offset & 3)) return -1;
  const float* p = reinterpret_cast<const float*>(mc) + elem_offset;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(dst)) & 15) return -2;
  rb::mc_reduce_f32_kernel<<<mc_grid(n / 4, max_ctas), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      p, reinterpret_cast<float*>(dst), n / 4, accumulate);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_mc_allreduce(void* mc, long long byte_offset, long long nbytes, int bf16, int max_ctas, void* stream) {
  if (!mc || nbytes <= 0 || (nbytes & 15) || (byte_offset & 15)) return -1;
  if (reinterpret_cast<uintptr_t>(mc) & 15) return -2;
  const long long first = byte_offset / 16, count = nbytes / 16;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (bf16) rb::mc_allreduce_kernel<true><<<mc_grid(count, max_ctas), 256, 0, s>>>(mc, first, count);
  else rb::mc_allreduce_kernel<false><<<mc_grid(count, max_ctas), 256, 0, s>>>(mc, first, count);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_mc_broadcast(const void* src, void* mc, long long byte_offset, long long nbytes, int max_ctas, void* stream) {
  if (!src || !mc || nbytes <= 0 || (nbytes & 15) || (byte_offset & 15)) return -1;
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(mc)) & 15) return -2;
  rb::mc_broadcast_kernel<<<mc_grid(nbytes / 16, max_ctas), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(src), reinterpret_cast<uint8_t*>(mc) + byte_offset, nbytes / 16);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_tp_allreduce_mc(const void* mc_stage, void* const* pad_ptrs_dev, const void* local_pad, int world, int rank, int channel,
                              const unsigned int* epoch_dev, int limit_ms, const void* residual, void* out, int rows, int cols,
                              void* stream) {
  if (!mc_stage || !pad_ptrs_dev || !local_pad || !epoch_dev || !out || world < 1 || world > 8 || rank < 0 || rank >= world) return -1;
  if (rows <= 0 || cols <= 0 || (cols % 8) || channel < 0 || limit_ms <= 0) return -1;
  if ((reinterpret_cast<uintptr_t>(mc_stage) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(residual)) & 15) return -2;
  const long long n8 = static_cast<long long>(rows) * (cols / 8);
  rb::tp_allreduce_mc_kernel<<<mc_grid(n8, 148 * 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      mc_stage, pad_ptrs_dev, reinterpret_cast<const unsigned int*>(local_pad), world, rank, channel, epoch_dev,
      static_cast<unsigned long long>(limit_ms) * 1000000ull, reinterpret_cast<const __nv_bfloat16*>(residual),
      reinterpret_cast<__nv_bfloat16*>(out), n8, rbhost::status_ptr());
  return static_cast<int>(cudaGetLastError());
}
