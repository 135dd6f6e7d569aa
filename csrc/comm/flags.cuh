// Flag primitives of the peer-memory communication kernels: system-scope release stores and acquire loads on u32
// words of a (possibly peer-mapped) signal pad, and the bounded wait built on them.
#pragma once
#include "rb_common.cuh"

namespace rb {

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait on `world` flags of one channel of the local pad.  One thread polls; returns false on expiry.
__device__ __forceinline__ bool wait_flags(const unsigned int* pad, int world, int channel, unsigned int value,
                                           unsigned long long limit_ns, unsigned int* status, unsigned int where) {
  const unsigned int* f = pad + channel * world;
  const unsigned long long t0 = globaltimer_ns();
  for (int r = 0; r < world; ++r) {
    while (true) {
      const unsigned int v = ld_acquire_sys(f + r);
      if (static_cast<int>(v - value) >= 0) break;     // wrap-safe "v >= value"
      if (globaltimer_ns() - t0 > limit_ns) {
        status_set(status, kStatusFlagTimeout, where);
        return false;
      }
      __nanosleep(200);
    }
  }
  return true;
}


// Same wait, for a value that may lie before the start of the sequence (value computed as epoch + delta <= 0 passes).
__device__ __forceinline__ bool wait_flags_from(const unsigned int* pad, int world, int channel, long long value,
                                                unsigned long long limit_ns, unsigned int* status, unsigned int where) {
  if (value <= 0) return true;
  return wait_flags(pad, world, channel, static_cast<unsigned int>(value), limit_ns, status, where);
}

}  // namespace rb
