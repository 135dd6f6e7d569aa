// Peer-memory communication kernels (NVLink P2P loads / stores from inside the kernels; no TMA multicast,
// no multimem in this file).  See symm.h for the protocol.
//
// Replaces the reference's host-slice collectives and its one-blocking-all-reduce-per-parameter step
// (crates/distributed/src/lib.rs:180-209,378-386), its ZeRO broadcast-per-parameter (crates/distributed/src/zero.rs:104-123)
// and the placeholder FSDP reduce-scatter / gather (crates/distributed/src/fsdp.rs:252-338).
#include "symm.h"

#include <string.h>

#include "rb_common.cuh"
#include "flags.cuh"

namespace rb {

constexpr int kSignalSlots = 64;   // channels per pad = kSignalSlots / world is never needed: pad is [channel][world]

__global__ void signal_all_kernel(void* const* pad_ptrs, int world, int my_rank, int channel, unsigned int value) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();   // everything this stream wrote before is visible before the flag
    st_release_sys(reinterpret_cast<unsigned int*>(pad_ptrs[r]) + channel * world + my_rank, value);
  }
}

__global__ void wait_all_kernel(const unsigned int* pad, int world, int channel, unsigned int value,
                                unsigned long long limit_ns, unsigned int* status) {
  if (threadIdx.x == 0) wait_flags(pad, world, channel, value, limit_ns, status, 100 + channel);
}

// ------------------------------------------------------------------------------------------------------------
// Phase 1: reduce this rank's shard over all peers, publish the partial norm.
// ------------------------------------------------------------------------------------------------------------
constexpr int kZeroThreads = 256;
constexpr int kMaxWorld = 16;

struct ZeroDev {
  const float* grads[kMaxWorld];
  __nv_bfloat16* lowp[kMaxWorld];
  unsigned int* pads[kMaxWorld];
  float* norms[kMaxWorld];
};

// The [world] pointer tables are device arrays owned by the caller's communicator; every CTA copies them into
// shared memory.  Nothing about them is cached on the host, so a communicator that is closed and another one that
// is created later in the same process never see each other's (unmapped) peer addresses.
__device__ __forceinline__ void load_tables(ZeroDev& d, const RbZeroArgs& a) {
  const int r = threadIdx.x;
  if (r < a.world) {
    d.grads[r] = reinterpret_cast<const float*>(a.grad_ptrs_dev[r]);
    d.lowp[r] = reinterpret_cast<__nv_bfloat16*>(a.lowp_ptrs_dev[r]);
    d.pads[r] = reinterpret_cast<unsigned int*>(a.pad_ptrs_dev[r]);
    d.norms[r] = reinterpret_cast<float*>(a.norm_ptrs_dev[r]);
  }
}

// Two u32 counters ("last CTA" election of the two kernels) live behind the per-CTA partial sums in the caller's
// scratch: partials[kZeroCounterSlot], partials[kZeroCounterSlot + 1].  They start at zero and are reset by the last CTA.
constexpr int kZeroCounterSlot = 1536;
constexpr int kZeroMaxGrid = 1024;

__global__ void __launch_bounds__(kZeroThreads)
zero_reduce_kernel(RbZeroArgs a, unsigned int* status) {
  __shared__ ZeroDev d;
  __shared__ int ok_sh;
  __shared__ float red[kZeroThreads / 32];
  load_tables(d, a);
  if (threadIdx.x == 0)
    ok_sh = wait_flags(reinterpret_cast<const unsigned int*>(a.local_pad), a.world, 0, a.epoch,
                       static_cast<unsigned long long>(a.limit_ms) * 1000000ull, status, 10) ? 1 : 0;
  __syncthreads();
  const bool ok = ok_sh != 0;
  float sq = 0.f;
  if (ok) {
    const long long n4 = a.shard_len / 4;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
      // All peer loads of an element are issued back to back (up to eight requests in flight per thread, spread over
      // all the peers at once, so no GPU is everybody's first target), then summed in rank order: the value does not
      // depend on timing.
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r0 = 0; r0 < a.world; r0 += 8) {
        float4 g[8];
        const int nr = min(8, a.world - r0);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < nr) g[j] = *(reinterpret_cast<const float4*>(d.grads[r0 + j] + a.shard_off) + i);   // peer load over NVLink
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < nr) { acc.x += g[j].x; acc.y += g[j].y; acc.z += g[j].z; acc.w += g[j].w; }
      }
      reinterpret_cast<float4*>(a.grad_shard)[i] = acc;
      sq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < kZeroThreads / 32; ++w) t += red[w];
    a.partials[blockIdx.x] = t;
    __threadfence();
    unsigned int* block_counter = reinterpret_cast<unsigned int*>(a.partials + kZeroCounterSlot);
    const unsigned int done = atomicAdd(block_counter, 1u);
    if (done == gridDim.x - 1) {
      // last CTA: fold the per-CTA partials in index order and publish to every rank
      __threadfence();
      float tot = 0.f;
      for (unsigned int b = 0; b < gridDim.x; ++b) tot += reinterpret_cast<volatile float*>(a.partials)[b];
      for (int r = 0; r < a.world; ++r) d.norms[r][a.rank] = tot;
      __threadfence_system();
      for (int r = 0; r < a.world; ++r) st_release_sys(d.pads[r] + 1 * a.world + a.rank, a.epoch);
      *block_counter = 0;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------
// Phase 2: AdamW on the shard, push bf16 parameters to every rank.
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kZeroThreads)
zero_adam_push_kernel(RbZeroArgs a, unsigned int* status) {
  __shared__ ZeroDev d;
  __shared__ int ok_sh;
  __shared__ float coef_sh;
  load_tables(d, a);
  if (threadIdx.x == 0) {
    const bool ok = wait_flags(reinterpret_cast<const unsigned int*>(a.local_pad), a.world, 1, a.epoch,
                               static_cast<unsigned long long>(a.limit_ms) * 1000000ull, status, 11);
    float coef = 1.f;
    if (ok && a.max_grad_norm > 0.f) {
      float tot = 0.f;
      for (int r = 0; r < a.world; ++r) tot += reinterpret_cast<volatile float*>(a.norm_slots)[r];
      const float c = a.max_grad_norm / (sqrtf(tot) + 1e-6f);
      if (c < 1.f) coef = c;
    }
    ok_sh = ok ? 1 : 0;
    coef_sh = coef;
  }
  __syncthreads();
  if (ok_sh) {
    const float coef = coef_sh;
    const float inv_bc1 = 1.f / a.bc1, inv_bc2 = 1.f / a.bc2;
    const long long n4 = a.shard_len / 4;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
      const float4 g4 = reinterpret_cast<const float4*>(a.grad_shard)[i];
      float4 p4 = reinterpret_cast<float4*>(a.master)[i];
      float4 m4 = reinterpret_cast<float4*>(a.m)[i];
      float4 v4 = reinterpret_cast<float4*>(a.v)[i];
      float g[4] = {g4.x, g4.y, g4.z, g4.w}, p[4] = {p4.x, p4.y, p4.z, p4.w};
      float m[4] = {m4.x, m4.y, m4.z, m4.w}, v[4] = {v4.x, v4.y, v4.z, v4.w};
      const float wd = (a.shard_off + i * 4 < a.decay_end) ? a.weight_decay : 0.f;   // groups are 128-aligned
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = g[j] * coef;
        m[j] = a.beta1 * m[j] + (1.f - a.beta1) * gj;
        v[j] = a.beta2 * v[j] + (1.f - a.beta2) * gj * gj;
        const float upd = (m[j] * inv_bc1) / (sqrtf(v[j] * inv_bc2) + a.eps) + wd * p[j];
        p[j] -= a.lr * upd;
      }
      reinterpret_cast<float4*>(a.master)[i] = make_float4(p[0], p[1], p[2], p[3]);
      reinterpret_cast<float4*>(a.m)[i] = make_float4(m[0], m[1], m[2], m[3]);
      reinterpret_cast<float4*>(a.v)[i] = make_float4(v[0], v[1], v[2], v[3]);
      uint2 o;
      o.x = pack_bf16x2(p[0], p[1]);
      o.y = pack_bf16x2(p[2], p[3]);
#pragma unroll 1
      for (int j = 0; j < a.world; ++j) {   // the all-gather: a direct store into every rank's working copy
        const int r = (a.rank + 1 + j) % a.world;
        *reinterpret_cast<uint2*>(d.lowp[r] + a.shard_off + i * 4) = o;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    unsigned int* block_counter = reinterpret_cast<unsigned int*>(a.partials + kZeroCounterSlot) + 1;
    const unsigned int done = atomicAdd(block_counter, 1u);
    if (done == gridDim.x - 1) {
      __threadfence_system();
      for (int r = 0; r < a.world; ++r) st_release_sys(d.pads[r] + 2 * a.world + a.rank, a.epoch);
      *block_counter = 0;
    }
  }
}

// out[r, :] = sum_s slots[s][r, :] (+ residual[r, :]), s ascending: the tail of the fused GEMM -> reduce-scatter.
__global__ void __launch_bounds__(256)
tp_reduce_slots_kernel(const __nv_bfloat16* __restrict__ slots, int world, long long slot_elems,
                       const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out) {
  const long long n8 = slot_elems / 8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (residual) {
      const uint4 u = reinterpret_cast<const uint4*>(residual)[i];
      const uint32_t* pu = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(pu[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
    }
    for (int s = 0; s < world; ++s) {
      const uint4 u = reinterpret_cast<const uint4*>(slots + s * slot_elems)[i];
      const uint32_t* pu = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(pu[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// One-shot all-reduce / all-gather over symmetric staging buffers (see symm.h).  Every CTA waits for the flags
// itself, so no grid-wide barrier is needed; CTA 0 raises this rank's flags before waiting.
__global__ void __launch_bounds__(256)
tp_allreduce_kernel(void* const* __restrict__ stage_ptrs, void* const* __restrict__ pad_ptrs,
                    const unsigned int* __restrict__ local_pad, int world, int rank, int channel, unsigned int epoch,
                    const unsigned int* __restrict__ epoch_dev, unsigned long long limit_ns,
                    const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out, int rows, int cols,
                    int gather, unsigned int* status) {
  __shared__ int ok_s;
  // A call captured in a CUDA graph cannot carry its epoch as a launch argument: it reads the counter that an
  // earlier kernel of the same stream has advanced.
  if (epoch_dev != nullptr) epoch = *epoch_dev;
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned int*>(pad_ptrs[threadIdx.x]) + channel * world + rank, epoch);
  }
  if (threadIdx.x == 0) ok_s = wait_flags(local_pad, world, channel, epoch, limit_ns, status, 120 + channel) ? 1 : 0;
  __syncthreads();
  if (!ok_s) return;
  const int c8 = cols / 8;
  const long long n8 = static_cast<long long>(rows) * c8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    if (gather) {
      const long long r = i / c8, c = i - r * c8;
      for (int s = 0; s < world; ++s) {
        const uint4 v = reinterpret_cast<const uint4*>(stage_ptrs[s])[i];
        reinterpret_cast<uint4*>(out + (r * world + s) * static_cast<long long>(cols))[c] = v;
      }
      continue;
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (residual) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(residual) + i);
      const uint32_t* pu = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(pu[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
    }
    for (int s = 0; s < world; ++s) {
      const uint4 u = reinterpret_cast<const uint4*>(stage_ptrs[s])[i];
      const uint32_t* pu = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(pu[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

}  // namespace rb

RB_API void* rb_symm_alloc(long long bytes) {
  void* p = nullptr;
  if (bytes <= 0 || cudaMalloc(&p, static_cast<size_t>(bytes)) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, static_cast<size_t>(bytes));
  cudaDeviceSynchronize();
  return p;
}
RB_API int rb_symm_free(void* ptr) { return static_cast<int>(cudaFree(ptr)); }
RB_API int rb_ipc_export(void* ptr, unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return static_cast<int>(e);
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
RB_API void* rb_ipc_import(const unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}
RB_API int rb_ipc_close(void* ptr) { return static_cast<int>(cudaIpcCloseMemHandle(ptr)); }

RB_API int rb_signal_all(void* const* pad_ptrs_dev, int world, int my_rank, int channel, unsigned int value, void* stream_v) {
  if (world < 1 || world > 32 || channel < 0 || (channel + 1) * world > rb::kSignalSlots * 4) return -1;
  rb::signal_all_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(pad_ptrs_dev, world, my_rank, channel, value);
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_wait_all(const void* local_pad, int world, int channel, unsigned int value, int limit_ms, void* stream_v) {
  if (world < 1 || world > 32 || channel < 0) return -1;
  rb::wait_all_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const unsigned int*>(local_pad), world, channel, value,
      static_cast<unsigned long long>(limit_ms > 0 ? limit_ms : 2000) * 1000000ull, rbhost::status_ptr());
  return static_cast<int>(cudaGetLastError());
}

static int zero_check(const RbZeroArgs* a) {
  if (!a || a->shard_len <= 0 || (a->shard_len % 4) || (a->shard_off % 4)) return -1;
  if (a->world < 1 || a->world > rb::kMaxWorld || a->rank < 0 || a->rank >= a->world) return -1;
  if (!a->grad_ptrs_dev || !a->lowp_ptrs_dev || !a->pad_ptrs_dev || !a->norm_ptrs_dev || !a->partials) return -1;
  return 0;
}

RB_API int rb_zero_reduce(const RbZeroArgs* a, void* stream_v) {
  const int rc = zero_check(a);
  if (rc != 0) return rc;
  int grid = rbhost::device_sm_count() * 2;
  if (grid > rb::kZeroMaxGrid) grid = rb::kZeroMaxGrid;
  rb::zero_reduce_kernel<<<grid, rb::kZeroThreads, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a, rbhost::status_ptr());
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_zero_adam_push(const RbZeroArgs* a, void* stream_v) {
  const int rc = zero_check(a);
  if (rc != 0) return rc;
  int grid = rbhost::device_sm_count() * 2;
  if (grid > rb::kZeroMaxGrid) grid = rb::kZeroMaxGrid;
  rb::zero_adam_push_kernel<<<grid, rb::kZeroThreads, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a, rbhost::status_ptr());
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_tp_reduce_slots(const void* slots, int world, long long slot_elems, const void* residual, void* out,
                              void* stream_v) {
  if (world < 1 || slot_elems <= 0 || (slot_elems % 8)) return -1;
  long long blocks = (slot_elems / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  rb::tp_reduce_slots_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const __nv_bfloat16*>(slots), world, slot_elems, reinterpret_cast<const __nv_bfloat16*>(residual),
      reinterpret_cast<__nv_bfloat16*>(out));
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_tp_allreduce(void* const* stage_ptrs_dev, void* const* pad_ptrs_dev, const void* local_pad, int world,
                           int rank, int channel, unsigned int epoch, const unsigned int* epoch_dev, int limit_ms,
                           const void* residual, void* out, int rows, int cols, int gather, void* stream_v) {
  if (!stage_ptrs_dev || !pad_ptrs_dev || !local_pad || !out || world < 1 || world > 8 || rank < 0 || rank >= world) return -1;
  if (rows <= 0 || cols <= 0 || (cols % 8) || channel < 0 || limit_ms <= 0) return -1;
  const long long n8 = static_cast<long long>(rows) * (cols / 8);
  long long blocks = (n8 + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  rb::tp_allreduce_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      stage_ptrs_dev, pad_ptrs_dev, reinterpret_cast<const unsigned int*>(local_pad), world, rank, channel, epoch, epoch_dev,
      static_cast<unsigned long long>(limit_ms) * 1000000ull, reinterpret_cast<const __nv_bfloat16*>(residual),
      reinterpret_cast<__nv_bfloat16*>(out), rows, cols, gather, rbhost::status_ptr());
  return static_cast<int>(cudaGetLastError());
}
