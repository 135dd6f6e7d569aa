// ZeRO-3 data plane over NVLink peer memory (see zero3.h for the protocol).  Plain peer loads / stores only.
//
// What this replaces in the reference: FSDP's gather-before-compute / reduce-scatter-after-backward, which there are
// host loops over a simulated process group (crates/distributed/src/fsdp.rs:238-249 forward gather, :252-278 gather,
// :323-338 reduce-scatter, :199-210 shard geometry), and the blocking all-reduce per parameter after backward
// (crates/distributed/src/lib.rs:378-386).  Here each bucket is moved by one kernel on a side stream while the tensor
// cores work on the neighbouring layer.
#include "zero3.h"

#include "flags.cuh"
#include "rb_common.cuh"

namespace rb {

constexpr int kZ3Threads = 256;
constexpr int kZ3MaxWorld = 16;
constexpr int kZ3MaxBuckets = 256;

__global__ void epoch_advance_kernel(unsigned int* p) {
  if (threadIdx.x == 0) *p += 1u;
}

// ---------------------------------------------------------------------------------------------------------------
// all-gather of one bucket's parameters (pull)
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kZ3Threads) zero3_gather_kernel(RbZero3Gather a, unsigned int* status) {
  // Shared memory is kept to one word: this kernel is meant to run beside GEMM CTAs that take almost all of an SM's
  // shared memory, and fits in what they leave.
  __shared__ int ok_sh;
  if (threadIdx.x == 0)
    ok_sh = wait_flags_from(reinterpret_cast<const unsigned int*>(a.local_pad), a.world, a.channel,
                            static_cast<long long>(*a.epoch_dev), static_cast<unsigned long long>(a.limit_ms) * 1000000ull,
                            status, 300) ? 1 : 0;
  __syncthreads();
  if (!ok_sh) return;
  const long long n8 = a.n_per_rank / 8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  uint4* dst = reinterpret_cast<uint4*>(a.dst);
  // Peers are visited starting with the next rank, so that at any moment the ranks pull from different GPUs.
  for (int j = 0; j < a.world; ++j) {
    const int r = (a.rank + 1 + j) % a.world;
    const uint4* s = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.lowp_ptrs_dev[r]) + a.shard_off);
    uint4* d = dst + r * n8;
    long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n8; i += 4 * stride) {          // four independent 16-byte requests in flight per thread
      const uint4 v0 = s[i], v1 = s[i + stride], v2 = s[i + 2 * stride], v3 = s[i + 3 * stride];
      d[i] = v0; d[i + stride] = v1; d[i + 2 * stride] = v2; d[i + 3 * stride] = v3;
    }
    for (; i < n8; i += stride) d[i] = s[i];
  }
}

// ---------------------------------------------------------------------------------------------------------------
// reduce-scatter of one bucket's gradients (pull), accumulated into the gradient shard
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kZ3Threads) zero3_reduce_kernel(RbZero3Reduce a, unsigned int* status) {
  __shared__ int ok_sh;                    // one word of shared memory only (see the gather kernel)
  const unsigned int epoch = *a.epoch_dev;
  // This kernel is stream-ordered after the kernels that wrote this rank's gradients of the bucket: tell every peer.
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned int*>(a.pad_ptrs_dev[threadIdx.x]) + a.ready_channel * a.world + a.rank, epoch);
  }
  if (threadIdx.x == 0)
    ok_sh = wait_flags(reinterpret_cast<const unsigned int*>(a.local_pad), a.world, a.ready_channel, epoch,
                       static_cast<unsigned long long>(a.limit_ms) * 1000000ull, status, 310) ? 1 : 0;
  __syncthreads();
  if (ok_sh) {
    const long long n4 = a.n_per_rank / 4;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    float4* dst = reinterpret_cast<float4*>(a.shard_dst);
    const long long my_off = static_cast<long long>(a.rank) * a.n_per_rank;
    const float4* src[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      src[j] = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.grad_ptrs_dev[j < a.world ? j : 0]) + my_off);
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
      // all peers' values are requested back to back, then added in rank order: independent of timing
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r0 = 0; r0 < a.world; r0 += 8) {
        float4 g[8];
        const int nr = min(8, a.world - r0);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < nr)
            g[j] = r0 == 0 ? src[j][i]
                           : (reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.grad_ptrs_dev[r0 + j]) + my_off))[i];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < nr) { acc.x += g[j].x; acc.y += g[j].y; acc.z += g[j].z; acc.w += g[j].w; }
      }
      if (a.accumulate) {
        const float4 o = dst[i];
        acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
      }
      dst[i] = acc;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int done = atomicAdd(a.counter, 1u);
    if (done == gridDim.x - 1) {
      // every CTA of this rank has finished reading the peers' buffers: they may overwrite them
      __threadfence_system();
      for (int r = 0; r < a.world; ++r)
        st_release_sys(reinterpret_cast<unsigned int*>(a.pad_ptrs_dev[r]) + a.consumed_channel * a.world + a.rank, epoch);
      *a.counter = 0;
    }
  }
}

__global__ void zero3_signal_kernel(void* const* pad_ptrs, int world, int rank, int channel, const unsigned int* epoch_dev) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned int*>(pad_ptrs[r]) + channel * world + rank, *epoch_dev);
  }
}

__global__ void __launch_bounds__(kZ3Threads) zero3_sum_kernel(RbZero3Sum a) {
  const long long n4 = a.n / 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  float4* dst = reinterpret_cast<float4*>(a.dst);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r0 = 0; r0 < a.num_src; r0 += 8) {
      float4 g[8];
      const int nr = min(8, a.num_src - r0);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < nr) g[j] = reinterpret_cast<const float4*>(a.src[r0 + j])[i];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < nr) { acc.x += g[j].x; acc.y += g[j].y; acc.z += g[j].z; acc.w += g[j].w; }
    }
    if (a.accumulate) {
      const float4 o = dst[i];
      acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
    }
    dst[i] = acc;
  }
}

__global__ void zero3_wait_kernel(const unsigned int* pad, int world, int channel, const unsigned int* epoch_dev, int delta,
                                  unsigned long long limit_ns, unsigned int* status) {
  if (threadIdx.x == 0)
    wait_flags_from(pad, world, channel, static_cast<long long>(*epoch_dev) + delta, limit_ns, status, 320);
}

// ---------------------------------------------------------------------------------------------------------------
// step tail: norm / loss exchange, clip, AdamW on the owned slices
// ---------------------------------------------------------------------------------------------------------------
__global__ void zero3_publish_kernel(RbZero3Step a) {
  const int r = threadIdx.x;
  if (r < a.world) {
    float* slots = reinterpret_cast<float*>(a.slots_ptrs_dev[r]);
    slots[a.rank] = *a.sumsq_local;
    slots[a.world + a.rank] = *a.loss_local;
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned int*>(a.pad_ptrs_dev[r]) + a.norm_channel * a.world + a.rank, a.step);
  }
}

__global__ void __launch_bounds__(kZ3Threads) zero3_adam_kernel(RbZero3Step a, unsigned int* status) {
  __shared__ int ok_sh;
  __shared__ float coef_sh;
  __shared__ long long start_sh[kZ3MaxBuckets + 1];
  __shared__ long long decay_sh[kZ3MaxBuckets];
  for (int b = threadIdx.x; b < a.num_buckets; b += blockDim.x) {
    start_sh[b] = a.bucket_shard_start[b];
    decay_sh[b] = a.bucket_decay_count[b];
  }
  if (threadIdx.x == 0) {
    start_sh[a.num_buckets] = a.shard_len;
    const bool ok = wait_flags(reinterpret_cast<const unsigned int*>(a.local_pad), a.world, a.norm_channel, a.step,
                               static_cast<unsigned long long>(a.limit_ms) * 1000000ull, status, 330);
    float coef = 1.f;
    if (ok) {
      float tot = 0.f, loss = 0.f;
      for (int r = 0; r < a.world; ++r) {
        tot += reinterpret_cast<const volatile float*>(a.local_slots)[r];
        loss += reinterpret_cast<const volatile float*>(a.local_slots)[a.world + r];
      }
      if (a.max_grad_norm > 0.f) {
        const float c = a.max_grad_norm / (sqrtf(tot) + 1e-6f);
        if (c < 1.f) coef = c;
      }
      if (blockIdx.x == 0 && a.loss_out) *a.loss_out = loss * a.loss_scale;
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
    __nv_bfloat16* lowp = reinterpret_cast<__nv_bfloat16*>(a.lowp_shard);
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
      const long long idx = i * 4;
      int lo = 0, hi = a.num_buckets - 1;        // last bucket whose first shard element is <= idx
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (start_sh[mid] <= idx) lo = mid; else hi = mid - 1;
      }
      const float wd = (idx - start_sh[lo] < decay_sh[lo]) ? a.weight_decay : 0.f;   // boundaries are multiples of 4
      const float4 g4 = reinterpret_cast<const float4*>(a.grad)[i];
      const float4 p4 = reinterpret_cast<const float4*>(a.master)[i];
      const float4 m4 = reinterpret_cast<const float4*>(a.m)[i];
      const float4 v4 = reinterpret_cast<const float4*>(a.v)[i];
      float g[4] = {g4.x, g4.y, g4.z, g4.w}, p[4] = {p4.x, p4.y, p4.z, p4.w};
      float m[4] = {m4.x, m4.y, m4.z, m4.w}, v[4] = {v4.x, v4.y, v4.z, v4.w};
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
      *reinterpret_cast<uint2*>(lowp + idx) = o;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int done = atomicAdd(a.counter, 1u);
    if (done == gridDim.x - 1) {
      // the whole shard of this rank is written: publish "parameters of step `step` are ready"
      __threadfence_system();
      *a.step_epoch_dev = a.step;
      for (int r = 0; r < a.world; ++r)
        st_release_sys(reinterpret_cast<unsigned int*>(a.pad_ptrs_dev[r]) + a.params_channel * a.world + a.rank, a.step);
      *a.counter = 0;
    }
  }
}

}  // namespace rb

namespace {
int block_threads(int threads) { return (threads == 64 || threads == 128) ? threads : rb::kZ3Threads; }

int clamp_grid(long long work_items, int max_ctas) {
  long long blocks = (work_items + rb::kZ3Threads - 1) / rb::kZ3Threads;
  const int cap = max_ctas > 0 ? max_ctas : 64;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}
}  // namespace

RB_API int rb_epoch_advance(unsigned int* epoch_dev, void* stream_v) {
  if (!epoch_dev) return -1;
  rb::epoch_advance_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(epoch_dev);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_zero3_gather(const RbZero3Gather* a, void* stream_v) {
  if (!a || !a->lowp_ptrs_dev || !a->local_pad || !a->epoch_dev || !a->dst) return -1;
  if (a->world < 1 || a->world > rb::kZ3MaxWorld || a->rank < 0 || a->rank >= a->world) return -1;
  if (a->n_per_rank <= 0 || (a->n_per_rank % 8) || (a->shard_off % 8) || a->channel < 0 || a->limit_ms <= 0) return -1;
  if (reinterpret_cast<uintptr_t>(a->dst) & 15) return -2;
  const int grid = clamp_grid(a->n_per_rank / 8, a->max_ctas);
  rb::zero3_gather_kernel<<<grid, block_threads(a->threads), 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a, rbhost::status_ptr());
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_zero3_reduce(const RbZero3Reduce* a, void* stream_v) {
  if (!a || !a->grad_ptrs_dev || !a->pad_ptrs_dev || !a->local_pad || !a->epoch_dev || !a->shard_dst || !a->counter) return -1;
  if (a->world < 1 || a->world > rb::kZ3MaxWorld || a->rank < 0 || a->rank >= a->world) return -1;
  if (a->n_per_rank <= 0 || (a->n_per_rank % 4) || a->ready_channel < 0 || a->consumed_channel < 0 || a->limit_ms <= 0) return -1;
  if (reinterpret_cast<uintptr_t>(a->shard_dst) & 15) return -2;
  const int grid = clamp_grid(a->n_per_rank / 4, a->max_ctas);
  rb::zero3_reduce_kernel<<<grid, block_threads(a->threads), 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a, rbhost::status_ptr());
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_zero3_signal(void* const* pad_ptrs_dev, int world, int rank, int channel, const unsigned int* epoch_dev,
                           void* stream_v) {
  if (!pad_ptrs_dev || !epoch_dev || world < 1 || world > rb::kZ3MaxWorld || rank < 0 || rank >= world || channel < 0) return -1;
  rb::zero3_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(pad_ptrs_dev, world, rank, channel, epoch_dev);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_zero3_sum(const RbZero3Sum* a, void* stream_v) {
  if (!a || !a->dst || a->n <= 0 || (a->n % 4) || a->num_src < 1 || a->num_src > 16) return -1;
  for (int i = 0; i < a->num_src; ++i)
    if (!a->src[i] || (reinterpret_cast<uintptr_t>(a->src[i]) & 15)) return -2;
  if (reinterpret_cast<uintptr_t>(a->dst) & 15) return -2;
  long long blocks = (a->n / 4 + rb::kZ3Threads - 1) / rb::kZ3Threads;
  const long long cap = 4LL * rbhost::device_sm_count();
  if (blocks > cap) blocks = cap;
  rb::zero3_sum_kernel<<<static_cast<int>(blocks), rb::kZ3Threads, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_zero3_wait(const void* local_pad, int world, int channel, const unsigned int* epoch_dev, int delta,
                         int limit_ms, void* stream_v) {
  if (!local_pad || !epoch_dev || world < 1 || world > rb::kZ3MaxWorld || channel < 0 || delta > 0 || limit_ms <= 0) return -1;
  rb::zero3_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const unsigned int*>(local_pad), world, channel, epoch_dev, delta,
      static_cast<unsigned long long>(limit_ms) * 1000000ull, rbhost::status_ptr());
  return static_cast<int>(cudaGetLastError());
}

static int step_check(const RbZero3Step* a) {
  if (!a || !a->pad_ptrs_dev || !a->local_pad || !a->slots_ptrs_dev || !a->local_slots) return -1;
  if (a->world < 1 || a->world > rb::kZ3MaxWorld || a->rank < 0 || a->rank >= a->world || a->limit_ms <= 0) return -1;
  if (a->norm_channel < 0 || a->params_channel < 0 || a->step == 0) return -1;
  return 0;
}

RB_API int rb_zero3_publish(const RbZero3Step* a, void* stream_v) {
  const int rc = step_check(a);
  if (rc != 0) return rc;
  if (!a->sumsq_local || !a->loss_local) return -1;
  rb::zero3_publish_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_zero3_adam(const RbZero3Step* a, void* stream_v) {
  const int rc = step_check(a);
  if (rc != 0) return rc;
  if (!a->master || !a->m || !a->v || !a->grad || !a->lowp_shard || !a->step_epoch_dev || !a->counter) return -1;
  if (a->shard_len <= 0 || (a->shard_len % 4) || a->num_buckets < 1 || a->num_buckets > rb::kZ3MaxBuckets) return -1;
  if (!a->bucket_shard_start || !a->bucket_decay_count) return -1;
  int grid = rbhost::device_sm_count() * 2;
  const long long need = (a->shard_len / 4 + rb::kZ3Threads - 1) / rb::kZ3Threads;
  if (grid > need) grid = static_cast<int>(need);
  if (grid < 1) grid = 1;
  rb::zero3_adam_kernel<<<grid, rb::kZ3Threads, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a, rbhost::status_ptr());
  return static_cast<int>(cudaGetLastError());
}
