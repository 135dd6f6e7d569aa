// Host-side services shared by all kernels of this library: the per-device status buffer, the
// tensor-map cache and device queries.
#include <mutex>
#include <string.h>
#include <unordered_map>
#include <vector>

#include "rb_common.cuh"

namespace rbhost {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

struct Key {
  uint64_t v[8];
  bool operator==(const Key& o) const { return memcmp(v, o.v, sizeof(v)) == 0; }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    uint64_t h = 1469598103934665603ull;
    for (int i = 0; i < 8; ++i) {
      h ^= k.v[i];
      h *= 1099511628211ull;
    }
    return static_cast<size_t>(h);
  }
};
std::mutex g_mu;
std::unordered_map<Key, CUtensorMap*, KeyHash> g_cache;
}  // namespace

const CUtensorMap* get_tmap_2d(const void* base, int elem_bytes, uint64_t inner, uint64_t outer, uint64_t ld,
                               uint32_t box_inner, uint32_t box_outer, int swizzle128, int* err) {
  int dev = 0;
  cudaGetDevice(&dev);
  Key k;
  k.v[0] = reinterpret_cast<uint64_t>(base);
  k.v[1] = inner; k.v[2] = outer; k.v[3] = ld;
  k.v[4] = (static_cast<uint64_t>(box_inner) << 32) | box_outer;
  k.v[5] = static_cast<uint64_t>(elem_bytes); k.v[6] = static_cast<uint64_t>(swizzle128);
  k.v[7] = static_cast<uint64_t>(dev);
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_cache.find(k);
  if (it != g_cache.end()) return it->second;
  // The encode is a driver call and needs this thread to have the device's primary context bound; a thread that has
  // made no runtime call yet (an autograd worker) has none.  cudaSetDevice binds it and, unlike cudaFree(0), is legal
  // while a stream is being captured into a graph.
  {
    int cur = 0;
    if (cudaGetDevice(&cur) == cudaSuccess) cudaSetDevice(cur);
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) { if (err) *err = -10; return nullptr; }
  if (g_cache.size() > 65536) {   // bound the cache; maps are cheap to rebuild
    for (auto& kv : g_cache) delete kv.second;
    g_cache.clear();
  }
  CUtensorMap* m = new CUtensorMap;
  cuuint64_t gdim[2] = {inner, outer};
  cuuint64_t gstride[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
  CUresult r = fn(m, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    delete m;
    if (err) *err = -100 - static_cast<int>(r);
    return nullptr;
  }
  g_cache.emplace(k, m);
  return m;
}

// 4-D variant for [batch, seq, head, dim] views: dims / strides are given innermost first, strides in BYTES for
// dimensions 1..3 (dimension 0 is contiguous).
const CUtensorMap* get_tmap_4d(const void* base, int elem_bytes, const uint64_t dims[4], const uint64_t strides_bytes[3],
                               const uint32_t box[4], int swizzle128, int* err) {
  int dev = 0;
  cudaGetDevice(&dev);
  Key k;
  k.v[0] = reinterpret_cast<uint64_t>(base);
  k.v[1] = dims[0] | (dims[1] << 20) | (dims[2] << 40);
  k.v[2] = dims[3] | (static_cast<uint64_t>(box[0]) << 32) | (static_cast<uint64_t>(box[2]) << 44);
  k.v[3] = strides_bytes[0];
  k.v[4] = strides_bytes[1];
  k.v[5] = strides_bytes[2];
  k.v[6] = static_cast<uint64_t>(elem_bytes) | (static_cast<uint64_t>(swizzle128) << 8) | (4ull << 16) |
           (static_cast<uint64_t>(box[1]) << 24) | (static_cast<uint64_t>(box[3]) << 40);
  k.v[7] = static_cast<uint64_t>(dev);
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_cache.find(k);
  if (it != g_cache.end()) return it->second;
  // The encode is a driver call and needs this thread to have the device's primary context bound; a thread that has
  // made no runtime call yet (an autograd worker) has none.  cudaSetDevice binds it and, unlike cudaFree(0), is legal
  // while a stream is being captured into a graph.
  {
    int cur = 0;
    if (cudaGetDevice(&cur) == cudaSuccess) cudaSetDevice(cur);
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) { if (err) *err = -10; return nullptr; }
  CUtensorMap* m = new CUtensorMap;
  cuuint64_t gdim[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t gstride[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(m, dt, 4, const_cast<void*>(base), gdim, gstride, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    delete m;
    if (err) *err = -100 - static_cast<int>(r);
    return nullptr;
  }
  g_cache.emplace(k, m);
  return m;
}

int device_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

unsigned int* status_ptr() {
  static unsigned int* ptrs[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (ptrs[dev]) return ptrs[dev];
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    unsigned int* p = nullptr;
    if (cudaMalloc(&p, 4 * sizeof(unsigned int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 4 * sizeof(unsigned int));
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

}  // namespace rbhost

// Reads (and optionally clears) the status buffer of the current device.  Synchronises the device.
// out[0] = OR of status bits, out[1] = code of the wait that gave up.
RB_API int rb_status_read(unsigned int* out, int clear) {
  unsigned int* p = rbhost::status_ptr();
  if (!p) return -1;
  cudaError_t e = cudaMemcpy(out, p, 4 * sizeof(unsigned int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (clear && (out[0] | out[1])) cudaMemset(p, 0, 4 * sizeof(unsigned int));
  return 0;
}

// Allocates the status buffer (first call on a device allocates; do it before any stream capture).
RB_API int rb_init() { return rbhost::status_ptr() ? 0 : -1; }

// Bit 0: the library was compiled with -DRB_BOUNDS (index checks report through the status word).
RB_API int rb_build_flags() {
#ifdef RB_BOUNDS
  return 1;
#else
  return 0;
#endif
}

RB_API int rb_sm_count() { return rbhost::device_sm_count(); }
