// Helpers of the peer-memory ring / context-parallel attention (parallel/peer_ring.py): every rank publishes its
// K / V block in a symmetric buffer, the others pull it over NVLink on a side stream while the tensor cores work on
// the previous block, partial results are merged with their log-sum-exp, and the key / value gradients travel back
// as peer stores into the owner's receive slots.  The reference's ring never moves a block
// (crates/distributed/src/sequence_parallel.rs:360-369) and merges outputs as if they were logits (:327-349).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ring.h"

namespace {

__global__ void peer_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long n16) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  // four independent 16-byte loads in flight per thread: NVLink latency is several times that of local HBM
  for (; i + 3 * stride < n16; i += 4 * stride) {
    uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
  }
  for (; i < n16; i += stride) dst[i] = src[i];
}

// one thread per 8 consecutive elements of the head dimension
__global__ void attn_merge_kernel(float* __restrict__ o_acc, float* __restrict__ lse_acc, const uint4* __restrict__ o_new,
                                  const float* __restrict__ lse_new, int B, int S, int H, int D8, int first,
                                  long long total) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = t < total;
  long long li = 0;
  int d8 = 1;
  float lse = 0.f;
  bool write_lse = false;
  if (live) {
    d8 = (int)(t % D8);
    const long long row = t / D8;               // (b, s, h)
    const int h = (int)(row % H);
    const long long bs = row / H;
    const int s = (int)(bs % S);
    const int b = (int)(bs / S);
    li = ((long long)b * H + h) * S + s;
    const float ln = lse_new[li];
    const uint4 raw = o_new[t];
    const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float nv[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(v2[i]);
      nv[2 * i] = f.x; nv[2 * i + 1] = f.y;
    }
    float4* acc = reinterpret_cast<float4*>(o_acc + t * 8);
    if (first) {
      const bool dead = ln == -INFINITY;
      acc[0] = dead ? make_float4(0.f, 0.f, 0.f, 0.f) : make_float4(nv[0], nv[1], nv[2], nv[3]);
      acc[1] = dead ? make_float4(0.f, 0.f, 0.f, 0.f) : make_float4(nv[4], nv[5], nv[6], nv[7]);
      lse = ln;
      write_lse = true;
    } else if (ln != -INFINITY) {               // -inf: nothing of this row was visible in the block
      const float la = lse_acc[li];
      float wa, wb;
      if (la == -INFINITY) {
        wa = 0.f; wb = 1.f; lse = ln;
      } else {
        const float mx = fmaxf(la, ln);
        const float ea = __expf(la - mx), eb = __expf(ln - mx);
        lse = mx + __logf(ea + eb);
        wa = ea / (ea + eb); wb = eb / (ea + eb);
      }
      float4 a0 = acc[0], a1 = acc[1];
      a0.x = a0.x * wa + nv[0] * wb; a0.y = a0.y * wa + nv[1] * wb; a0.z = a0.z * wa + nv[2] * wb; a0.w = a0.w * wa + nv[3] * wb;
      a1.x = a1.x * wa + nv[4] * wb; a1.y = a1.y * wa + nv[5] * wb; a1.z = a1.z * wa + nv[6] * wb; a1.w = a1.w * wa + nv[7] * wb;
      acc[0] = a0; acc[1] = a1;
      write_lse = true;
    }
  }
  // the D8 threads of a row all read lse_acc[li] above; they sit in one block (blockDim.x is a multiple of D8 and
  // rows start on multiples of D8), so one barrier orders those reads before the single write below
  __syncthreads();
  if (live && write_lse && d8 == 0) lse_acc[li] = lse;
}

__global__ void ring_fold_kernel(const uint2* __restrict__ slots, int world, unsigned int mask, long long slot4,
                                 uint2* __restrict__ out) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < slot4; i += stride) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      if (!((mask >> r) & 1u)) continue;
      const uint2 raw = slots[(long long)r * slot4 + i];
      const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
      const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      s.x += lo.x; s.y += lo.y; s.z += hi.x; s.w += hi.y;
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(s.x, s.y), hi = __floats2bfloat162_rn(s.z, s.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    out[i] = o;
  }
}

}  // namespace

extern "C" int rb_peer_copy(void* dst, const void* src, long long bytes, int ctas, void* stream) {
  if (!dst || !src || bytes < 0 || (bytes & 15) || ((uintptr_t)dst & 15) || ((uintptr_t)src & 15)) return -1;
  if (bytes == 0) return 0;
  if (ctas < 0)                                 // copy engine instead of SMs
    return (int)cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)stream);
  if (ctas == 0) ctas = 32;
  const long long n16 = bytes / 16;
  const long long want = (n16 + 255) / 256;
  const int grid = (int)(want < ctas ? want : ctas);
  peer_copy_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((uint4*)dst, (const uint4*)src, n16);
  return (int)cudaGetLastError();
}

extern "C" int rb_attn_merge(float* o_acc, float* lse_acc, const void* o_new, const float* lse_new, int B, int S, int H,
                             int D, int first, void* stream) {
  if (!o_acc || !lse_acc || !o_new || !lse_new || B <= 0 || S <= 0 || H <= 0 || D <= 0 || (D & 7) || D > 256) return -1;
  const int D8 = D / 8;
  if (256 % D8) return -1;                      // rows must not straddle a block (see the kernel)
  const long long total = (long long)B * S * H * D8;
  const long long blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return -1;
  attn_merge_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(o_acc, lse_acc, (const uint4*)o_new, lse_new, B, S, H,
                                                                         D8, first, total);
  return (int)cudaGetLastError();
}

extern "C" int rb_ring_fold(const void* slots, int world, unsigned int mask, long long slot_elems, void* out, void* stream) {
  if (!slots || !out || world <= 0 || world > 32 || slot_elems <= 0 || (slot_elems & 3)) return -1;
  const long long slot4 = slot_elems / 4;
  long long blocks = (slot4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  ring_fold_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const uint2*)slots, world, mask, slot4, (uint2*)out);
  return (int)cudaGetLastError();
}
