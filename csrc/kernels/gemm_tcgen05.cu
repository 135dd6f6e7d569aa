// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, operands staged in
// shared memory by TMA, 128-byte swizzle), persistent over output tiles, warp-specialised:
//   warp 0      : TMA producer (one elected lane)
//   warp 1      : TMEM allocator + MMA issuer (one elected lane)
//   warps 2..5  : epilogue (TMEM -> registers -> fused epilogue -> global)
// TMEM holds two accumulator buffers, so the epilogue of tile i overlaps the main loop of tile i+1.
//
// D[M,N] = epilogue( A[M,K] * B[N,K]^T ).  Each operand is either "K-major" (the contraction
// dimension is the contiguous one, i.e. A stored [M,K] / B stored [N,K]) or "MN-major" (stored
// transposed, [K,M] / [K,N]).  The three combinations a linear layer needs are
//   forward  y  = x W^T      : A K-major,  B K-major
//   dgrad    dx = dy W       : A K-major,  B MN-major
//   wgrad    dW = dy^T x     : A MN-major, B MN-major
// so neither activations nor weights are ever transposed in memory.
//
// Replaces the reference's scalar 16x16 tiled matmul (crates/wgpu-backend/src/shaders.wgsl:571),
// its CPU linear (crates/ndarray-backend/src/lib.rs:478) and the fused_linear_bias{,_relu,_gelu}
// op sequences (crates/candle-backend/src/lib.rs:220-312).
#include "gemm_tcgen05.h"

#include <stdlib.h>
#include <string.h>

#include "rb_common.cuh"

namespace rb {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;   // 64 bf16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;
constexpr int kNumEpilogueWarps = 8;   // two groups of four: each group covers all 128 TMEM lanes and half of the columns
constexpr int kNumEpiThreads = kNumEpilogueWarps * 32;
constexpr int kNumThreads = 64 + kNumEpiThreads;

struct EpiParams {
  void* d;
  long long ldd;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  const __nv_bfloat16* aux_in;
  long long ld_aux_in;
  __nv_bfloat16* aux_out;
  long long ld_aux_out;
  int act;
  int out_f32;
  int accumulate;
  float alpha;
  int staged;   // 1: bf16 output goes through a per-warp shared-memory tile and leaves as whole 128/256-byte row segments;
                // 2: the same tile leaves through a TMA store (tensor maps tmD / tmAux; 64-column tiles only)
  const float* row_scale;   // fp32 [M] or nullptr: multiplies row i of the accumulator (8-bit operands: per-token scale)
  const float* col_scale;   // fp32 [N] or nullptr: multiplies column j (per-output-channel weight scale)
  int fp8_b_format;         // 8-bit operands: format of B in the instruction descriptor (0 = e4m3, 1 = e5m2); A is e4m3
};

// Grouped (mixture-of-experts) execution over a permuted token buffer whose expert segments are whole tiles.
//   mode 1: rows of A (and D) belong to experts; the expert of M-tile i is tile_expert[i], the number of M-tiles
//           is read from the device (*num_m_tiles).  B holds all experts stacked: expert e starts b_expert_rows
//           rows further (along N for a K-major B, along K for an MN-major B).
//   mode 2: one output matrix per expert (d + e * d_expert_stride); expert e contracts over the rows
//           [offsets[e], offsets[e+1]) of A and B (both MN-major).  An expert without tokens writes zeros.
struct GroupInfo {
  int mode;
  int num_experts;
  const int* tile_expert;
  const int* num_m_tiles;
  const int* offsets;
  int b_expert_rows;
  long long d_expert_stride;
  const unsigned int* tile_arrived;   // mode 1, optional: rows of A's 128-row tiles stored so far by the dispatching ranks
  const int* tile_expected;           //                    rows each tile has to receive before it may be read
};

// Fusion with tensor-parallel collectives over peer memory (NVLink loads / stores issued by this kernel).
//   mode 1 (all-gather -> GEMM): the A operand [M, K] is sharded by rows over `world` ranks.  This rank's rows are
//           already in a_full; the other ranks' 128-row tiles are copied from their (peer-mapped) shards into a_full by
//           the epilogue warps of all CTAs whenever they have no accumulator to drain, 4 rows at a time, each piece adding one to the tile's
//           counter; the TMA producer waits (bounded) until a remote tile's counter reaches epoch * 32 before loading
//           it.  Local tiles are scheduled first, so the transfer overlaps their math.
//   mode 3 (weight all-gather -> GEMM, the FSDP / ZeRO-3 case): the B operand [N, K] is sharded by rows over the
//           ranks; same pull-and-flag mechanism as mode 1 on 128-row blocks of B, with the tiles visited N-major
//           starting at this rank's own block of output columns.
//   mode 2 (GEMM -> reduce-scatter): the output rows are owned by ranks (rows_per_rank each).  The epilogue stores
//           every tile straight into the OWNER's receive slot for this rank (d_peer[owner] + rank slot), as whole
//           row segments through the staged store; tiles of the next rank come first and this rank's own last, so
//           at any time the ranks send to different peers.  A small kernel on the owner then folds the slots in
//           rank order.
struct PeerInfo {
  int mode, world, rank, rows_per_rank;
  const __nv_bfloat16* a_peer[8];
  __nv_bfloat16* a_full;
  unsigned int* ready;
  unsigned int epoch;
  __nv_bfloat16* d_peer[8];
};

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
constexpr int kCopyParts = 32;    // a remote 128-row block is pulled as 32 pieces of 4 rows, by different warps of different CTAs
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

template <int BLOCK_N, int STAGES>
struct SmemLayout {
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BLOCK_N * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem ptr, abort flag
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 4) * 8 + 16;
  // optional output staging (EpiParams::staged): per epilogue warp 32 rows x kStageCols bf16
  static constexpr int kStageCols = (BLOCK_N % 128 == 0) ? 64 : 32;
  static constexpr int kStagingOffset = (kTotal + 1023) & ~1023;   // 1024-byte aligned: the tiles are also TMA-store sources (128B swizzle)
  static constexpr int kStagingBytesPerWarp = 32 * kStageCols * 2;
  static constexpr int kTotalStaged = kStagingOffset + kNumEpilogueWarps * kStagingBytesPerWarp;
};

// Epilogue arithmetic on 32 consecutive accumulator columns of one output row (everything but the final store).
// STORE_AUX: write the pre-activation to aux_out from here (one 64-byte piece per thread).  PRE_ONLY: stop after
// the bias, leaving the pre-activation in v (the staged path writes it out itself, coalesced).
// POST_ONLY: v already holds the pre-activation; only the activation and the residual are applied.
template <bool STORE_AUX = true, bool PRE_ONLY = false, bool POST_ONLY = false>
__device__ __forceinline__ void epilogue_math(const EpiParams& ep, uint32_t (&r)[32], long long row, int col0, int N,
                                              float (&v)[32]) {
  const bool full = (col0 + 32 <= N);
  if (!POST_ONLY) {
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * ep.alpha;

  if (ep.row_scale != nullptr) {
    const float rs = __ldg(ep.row_scale + row);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= rs;
  }
  if (ep.col_scale != nullptr) {
    if (full) {
      const float4* cp = reinterpret_cast<const float4*>(ep.col_scale + col0);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 c = __ldg(cp + q);
        v[q * 4 + 0] *= c.x; v[q * 4 + 1] *= c.y; v[q * 4 + 2] *= c.z; v[q * 4 + 3] *= c.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < N) v[j] *= __ldg(ep.col_scale + col0 + j);
    }
  }

  if (ep.bias != nullptr) {
    if (full) {
      const uint4* bp = reinterpret_cast<const uint4*>(ep.bias + col0);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 b = __ldg(bp + q);
        float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
        v[q * 8 + 0] += f0.x; v[q * 8 + 1] += f0.y; v[q * 8 + 2] += f1.x; v[q * 8 + 3] += f1.y;
        v[q * 8 + 4] += f2.x; v[q * 8 + 5] += f2.y; v[q * 8 + 6] += f3.x; v[q * 8 + 7] += f3.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < N) v[j] += __bfloat162float(ep.bias[col0 + j]);
    }
  }

  }   // !POST_ONLY

  if (PRE_ONLY) return;

  if (ep.act == RB_ACT_GELU || ep.act == RB_ACT_RELU || ep.act == RB_ACT_SILU) {
    if (ep.aux_out != nullptr) {   // keep the pre-activation for the backward pass
      __nv_bfloat16* ap = ep.aux_out + row * ep.ld_aux_out + col0;
      if (!STORE_AUX) {
      } else if (full) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 o;
          o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]); o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
          o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]); o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
          reinterpret_cast<uint4*>(ap)[q] = o;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < N) ap[j] = __float2bfloat16(v[j]);
      }
      // The activation is applied to the unrounded fp32 value; the backward pass differentiates at the bf16-rounded
      // one it reads back (a relative difference of 2^-9 in the argument).  Rounding here as well costs two conversions
      // per element in an epilogue whose conversion and special-function work already exceeds the main loop at K = 768.
    }
    if (ep.act == RB_ACT_GELU) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = gelu_tanh_fast(v[j]);
    } else if (ep.act == RB_ACT_RELU) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = silu(v[j]);
    }
  } else if (ep.act == RB_ACT_DGELU || ep.act == RB_ACT_DRELU || ep.act == RB_ACT_DSILU || ep.act == RB_ACT_MUL) {
    // multiply by act'(aux_in) (or by aux_in itself for RB_ACT_MUL)
    const __nv_bfloat16* ap = ep.aux_in + row * ep.ld_aux_in + col0;
    float a[32];
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 b = __ldg(reinterpret_cast<const uint4*>(ap) + q);
        float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
        a[q * 8 + 0] = f0.x; a[q * 8 + 1] = f0.y; a[q * 8 + 2] = f1.x; a[q * 8 + 3] = f1.y;
        a[q * 8 + 4] = f2.x; a[q * 8 + 5] = f2.y; a[q * 8 + 6] = f3.x; a[q * 8 + 7] = f3.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) a[j] = (col0 + j < N) ? __bfloat162float(ap[j]) : 0.f;
    }
    if (ep.act == RB_ACT_DGELU) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= gelu_tanh_grad_fast(a[j]);
    } else if (ep.act == RB_ACT_DRELU) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = a[j] > 0.f ? v[j] : 0.f;
    } else if (ep.act == RB_ACT_DSILU) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= silu_grad(a[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= a[j];
    }
  }

  if (ep.residual != nullptr) {
    const __nv_bfloat16* rp = ep.residual + row * ep.ldr + col0;
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 b = __ldg(reinterpret_cast<const uint4*>(rp) + q);
        float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
        v[q * 8 + 0] += f0.x; v[q * 8 + 1] += f0.y; v[q * 8 + 2] += f1.x; v[q * 8 + 3] += f1.y;
        v[q * 8 + 4] += f2.x; v[q * 8 + 5] += f2.y; v[q * 8 + 6] += f3.x; v[q * 8 + 7] += f3.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < N) v[j] += __bfloat162float(rp[j]);
    }
  }

}

// Stores 32 consecutive columns of one output row from registers.
__device__ __forceinline__ void epilogue_store(const EpiParams& ep, float (&v)[32], long long row, int col0, int N) {
  const bool full = (col0 + 32 <= N);
  if (ep.out_f32) {
    float* dp = reinterpret_cast<float*>(ep.d) + row * ep.ldd + col0;
    if (full) {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float4 o = make_float4(v[q * 4 + 0], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
        if (ep.accumulate) {
          float4 old = reinterpret_cast<float4*>(dp)[q];
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        reinterpret_cast<float4*>(dp)[q] = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < N) dp[j] = ep.accumulate ? dp[j] + v[j] : v[j];
    }
  } else {
    __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(ep.d) + row * ep.ldd + col0;
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (ep.accumulate) {
          uint4 b = reinterpret_cast<uint4*>(dp)[q];
          float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
          v[q * 8 + 0] += f0.x; v[q * 8 + 1] += f0.y; v[q * 8 + 2] += f1.x; v[q * 8 + 3] += f1.y;
          v[q * 8 + 4] += f2.x; v[q * 8 + 5] += f2.y; v[q * 8 + 6] += f3.x; v[q * 8 + 7] += f3.y;
        }
        uint4 o;
        o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]); o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
        o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]); o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
        reinterpret_cast<uint4*>(dp)[q] = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < N) {
          float o = v[j];
          if (ep.accumulate) o += __bfloat162float(dp[j]);
          dp[j] = __float2bfloat16(o);
        }
    }
  }
}

__device__ __forceinline__ void epilogue_chunk(const EpiParams& ep, uint32_t (&r)[32], long long row, int col0, int N) {
  float v[32];
  epilogue_math(ep, r, row, col0, N, v);
  epilogue_store(ep, v, row, col0, N);
}

// FP8 = 1: both operands hold e4m3 bytes (K-major only).  A 128-byte swizzle row then carries 128 elements, so K, lda
// and ldb arrive halved (in units of two bytes) and only the TMA coordinates, which count elements, are doubled back.
template <int A_MN, int B_MN, int BLOCK_N, int STAGES, int FP8 = 0>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmAux, int M, int N,
                 int K, int group_m, int num_splits, int kb_per_split, long long d_split_stride, EpiParams ep,
                 GroupInfo grp, PeerInfo peer, unsigned int* status) {
  using L = SmemLayout<BLOCK_N, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle atoms need 1024-byte aligned tiles
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = smem_u32(bars + STAGES);
  const uint32_t bar_tfull = smem_u32(bars + 2 * STAGES);
  const uint32_t bar_tempty = smem_u32(bars + 2 * STAGES + 2);
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // TMEM allocations are powers of two >= 32 columns
  constexpr uint32_t kTmemCols = (2 * BLOCK_N <= 32) ? 32 : (2 * BLOCK_N <= 64) ? 64 : (2 * BLOCK_N <= 128) ? 128
                                 : (2 * BLOCK_N <= 256) ? 256 : 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, kNumEpilogueWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  int num_m = (M + kBlockM - 1) / kBlockM;
  if (grp.mode == 1) num_m = min(num_m, __ldg(grp.num_m_tiles));
  const int num_n = (N + BLOCK_N - 1) / BLOCK_N;
  const int num_tiles = num_m * num_n;
  const int num_kb_total = (K + kBlockK - 1) / kBlockK;
  const int group_size = group_m * num_n;
  // Work units: (split, tile).  With split-K every unit reduces its own K range into its own fp32 slab
  // d + split * d_split_stride; a second kernel folds the slabs in a fixed order.
  const int num_units = num_tiles * (grp.mode == 2 ? grp.num_experts : num_splits);

  // `outer` is the split index (split-K) or the expert index (grouped mode 2)
  auto decode_tile = [&](int unit, int& m_blk, int& n_blk, int& kb0, int& kb1, int& outer) {
    const int split = unit / num_tiles;
    const int tile = unit - split * num_tiles;
    outer = split;
    if (grp.mode == 2) {
      kb0 = __ldg(grp.offsets + split) / kBlockK;
      kb1 = __ldg(grp.offsets + split + 1) / kBlockK;
    } else {
      kb0 = split * kb_per_split;
      kb1 = min(num_kb_total, kb0 + kb_per_split);
    }
    const int group = tile / group_size;
    const int first_m = group * group_m;
    const int gm = min(group_m, num_m - first_m);
    const int in_group = tile - group * group_size;
    m_blk = first_m + in_group % gm;
    n_blk = in_group / gm;
    if (peer.mode == 1) {          // consumption order starts at this rank's own rows
      m_blk += peer.rank * (peer.rows_per_rank / kBlockM);
      if (m_blk >= num_m) m_blk -= num_m;
    } else if (peer.mode == 3) {   // N-major walk starting at this rank's own columns
      const int n_i = tile / num_m;
      m_blk = tile - n_i * num_m;
      n_blk = n_i + peer.rank * (peer.rows_per_rank / BLOCK_N);
      if (n_blk >= num_n) n_blk -= num_n;
    } else if (peer.mode == 2) {   // rows of the next rank first, this rank's own rows last
      m_blk += ((peer.rank + 1) % peer.world) * (peer.rows_per_rank / kBlockM);
      if (m_blk >= num_m) m_blk -= num_m;
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_units && ok; tile += gridDim.x) {
        int m_blk, n_blk, kb0, kb1, outer;
        decode_tile(tile, m_blk, n_blk, kb0, kb1, outer);
        // grouped mode 1: this M-tile's expert selects the slice of B
        int b_row_off = 0;
        if (grp.mode == 1) {
          const int e = __ldg(grp.tile_expert + m_blk);
          b_row_off = (e < 0 ? 0 : e) * grp.b_expert_rows;
        }
        if (grp.mode == 1 && grp.tile_arrived != nullptr) {
          // expert-parallel dispatch still in flight: this 128-row tile of A is complete once every rank has stored the
          // rows it routes here (counted with system-scope release adds by the dispatch kernels)
          const unsigned int want = static_cast<unsigned int>(__ldg(grp.tile_expected + m_blk));
          const unsigned long long t0 = globaltimer_ns();
          while (ld_acquire_sys_u32(grp.tile_arrived + m_blk) < want) {
            if (*abort_flag || globaltimer_ns() - t0 > kFlagWaitLimitNs) {
              *abort_flag = 1;
              status_set(status, kStatusFlagTimeout, 6);
              ok = false;
              break;
            }
            __nanosleep(100);
          }
          if (!ok) break;
          fence_proxy_async_all();
        }
        if (peer.mode == 1 || peer.mode == 3) {
          // remote 128-row blocks this tile reads: wait until the copy warps have landed all their pieces
          const int blk0 = peer.mode == 1 ? m_blk : n_blk * (BLOCK_N / 128);
          const int nblk = peer.mode == 1 ? 1 : BLOCK_N / 128;
          const unsigned int target = peer.epoch * kCopyParts;
          for (int bi = blk0; bi < blk0 + nblk && ok; ++bi) {
            if ((bi * 128) / peer.rows_per_rank == peer.rank) continue;
            const unsigned long long t0 = globaltimer_ns();
            while (static_cast<int>(ld_acquire_gpu(peer.ready + bi) - target) < 0) {
              if (*abort_flag || globaltimer_ns() - t0 > kFlagWaitLimitNs) {
                *abort_flag = 1;
                status_set(status, kStatusFlagTimeout, 5);
                ok = false;
                break;
              }
              __nanosleep(100);
            }
          }
          if (!ok) break;
          fence_proxy_async_all();     // the rows were written with ordinary stores; TMA reads them through the async proxy
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, status, 1)) { ok = false; break; }
          const uint32_t full = bar_full + 8 * s;
          mbar_arrive_expect_tx(full, L::kStageBytes);
          const uint32_t sa = smem_base + s * L::kStageBytes;
          const uint32_t sb = sa + L::kABytes;
          if (A_MN == 0) {
            tma_load_2d(sa, &tmA, kb * kBlockK * (FP8 ? 2 : 1), m_blk * kBlockM, full);
          } else {
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j)
              tma_load_2d(sa + j * (kBlockK * 128), &tmA, m_blk * kBlockM + j * 64, kb * kBlockK, full);
          }
          if (B_MN == 0) {
            tma_load_2d(sb, &tmB, kb * kBlockK * (FP8 ? 2 : 1), b_row_off + n_blk * BLOCK_N, full);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_N / 64; ++j)
              tma_load_2d(sb + j * (kBlockK * 128), &tmB, n_blk * BLOCK_N + j * 64, b_row_off + kb * kBlockK, full);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      const uint32_t idesc = FP8 ? (umma_idesc_e4m3(kBlockM, BLOCK_N) | (static_cast<uint32_t>(ep.fp8_b_format) << 10))
                                 : umma_idesc_bf16(kBlockM, BLOCK_N, A_MN, B_MN);
      uint32_t it = 0, t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_units && ok; tile += gridDim.x, ++t) {
        int m_blk, n_blk, kb0, kb1, outer;
        decode_tile(tile, m_blk, n_blk, kb0, kb1, outer);
        const uint32_t acc = t & 1, acc_ph = (t >> 1) & 1;
        if (!mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, abort_flag, status, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BLOCK_N;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, status, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + s * L::kStageBytes;
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            // K-major: 32 bytes per UMMA_K step inside the swizzle row; 8-row groups 1024 B apart.
            // MN-major: 16 k-rows of 128 B per step; 64-wide MN atoms kBlockK*128 B apart.
            const uint64_t da = A_MN ? umma_smem_desc_sw128(sa + k * (kUmmaK * 128), kBlockK * 128, 1024)
                                     : umma_smem_desc_sw128(sa + k * (kUmmaK * 2), 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc_sw128(sb + k * (kUmmaK * 128), kBlockK * 128, 1024)
                                     : umma_smem_desc_sw128(sb + k * (kUmmaK * 2), 16, 1024);
            if (FP8) umma_f8_ss(tmem_d, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
            else umma_bf16_ss(tmem_d, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit(bar_empty + 8 * s);   // frees the smem stage once these MMAs have read it
        }
        if (ok) umma_commit(bar_tfull + 8 * acc);   // accumulator complete
      }
    }
  } else {
    // -------------------------------------------------------------------- epilogue warps
    const int q = warp & 3;   // TMEM lane quarter this warp may read
    const int ew = warp - 2;  // 0..7
    const int cgrp = ew >> 2; // which half of the tile's columns this warp handles
    bool store_pending = false;   // a bulk tensor store of this warp's staging tile may still be reading it
    // ---- all-gather duty (peer modes 1 and 3): every epilogue warp of every CTA owns a strided share of the 16-row
    // pieces of the remote rows, in the order the tiles consume them.  A warp pulls pieces whenever its next
    // accumulator is not ready yet, and finishes its share after its last tile; nothing a piece needs ever waits.
    const bool gathers = peer.mode == 1 || peer.mode == 3;
    const int tpr = gathers ? peer.rows_per_rank / kBlockM : 0;
    const int num_blk = peer.mode == 1 ? num_m : N / kBlockM;          // 128-row blocks of the gathered operand
    const int remote_items = gathers ? (num_blk - tpr) * kCopyParts : 0;
    const int item_stride = gridDim.x * kNumEpilogueWarps;
    int next_item = blockIdx.x * kNumEpilogueWarps + ew;
    auto copy_one = [&]() {
      const int c = next_item / kCopyParts, part = next_item - c * kCopyParts;
      next_item += item_stride;
      int mt = c + tpr + peer.rank * tpr;                 // consumption order -> global block index
      while (mt >= num_blk) mt -= num_blk;
      const int owner = (mt * kBlockM) / peer.rows_per_rank;
      const long long row0 = static_cast<long long>(mt) * kBlockM + part * (kBlockM / kCopyParts);
      const uint4* src = reinterpret_cast<const uint4*>(peer.a_peer[owner] +
                                                        (row0 - static_cast<long long>(owner) * peer.rows_per_rank) * K);
      uint4* dst = reinterpret_cast<uint4*>(peer.a_full + row0 * K);
      const int total = (kBlockM / kCopyParts) * (K / 8);   // 16-byte chunks per piece
      int i = lane;
      for (; i + 7 * 32 < total; i += 8 * 32) {             // eight peer loads in flight per thread
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = src[i + u * 32];
#pragma unroll
        for (int u = 0; u < 8; ++u) dst[i + u * 32] = v[u];
      }
      for (; i < total; i += 32) dst[i] = src[i];
      __threadfence();
      __syncwarp();
      if (lane == 0) {
        fence_proxy_async_all();
        red_release_gpu_add(peer.ready + mt, 1u);
      }
      __syncwarp();
    };
    uint32_t t = 0;
    for (int tile = blockIdx.x; tile < num_units; tile += gridDim.x, ++t) {
      int m_blk, n_blk, kb0, kb1, outer;
      decode_tile(tile, m_blk, n_blk, kb0, kb1, outer);
      EpiParams epu = ep;
      if (num_splits > 1)
        epu.d = reinterpret_cast<float*>(ep.d) + static_cast<long long>(outer) * d_split_stride;
      if (grp.mode == 2) {
        if (ep.out_f32) epu.d = reinterpret_cast<float*>(ep.d) + static_cast<long long>(outer) * grp.d_expert_stride;
        else epu.d = reinterpret_cast<__nv_bfloat16*>(ep.d) + static_cast<long long>(outer) * grp.d_expert_stride;
      }
      if (peer.mode == 2) {
        // this tile's rows belong to `owner`; write into the owner's receive slot for this rank
        const int owner = (m_blk * kBlockM) / peer.rows_per_rank;
        epu.d = peer.d_peer[owner] + (static_cast<long long>(peer.rank) - owner) * peer.rows_per_rank * ep.ldd;
      }
      const bool empty_k = kb1 <= kb0;     // an expert without tokens: the accumulator was never written
      const uint32_t acc = t & 1, acc_ph = (t >> 1) & 1;
      while (next_item < remote_items && !mbar_test(bar_tfull + 8 * acc, acc_ph)) copy_one();
      if (!mbar_wait(bar_tfull + 8 * acc, acc_ph, abort_flag, status, 4)) break;
      tc_fence_after();
      const long long row = static_cast<long long>(m_blk) * kBlockM + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BLOCK_N;
      if (epu.staged) {
        // registers -> swizzled per-warp tile in shared memory -> whole row segments to global / peer memory
        constexpr int SC = L::kStageCols, CPR = SC / 8;           // staged columns, 16-byte chunks per row
        const uint32_t stg = smem_base + L::kStagingOffset + ew * L::kStagingBytesPerWarp;
        constexpr int NB = (BLOCK_N / 2) / SC;                    // column blocks per warp group
        const bool two_pass = epu.aux_out != nullptr &&
                              (epu.act == RB_ACT_GELU || epu.act == RB_ACT_RELU || epu.act == RB_ACT_SILU);
        if (SC == 64 && epu.staged == 2 && two_pass) {
          // One pass over the accumulator: the pre-activation is rounded to bf16, kept packed in registers for the 64
          // columns of a block and sent to aux_out by a bulk store; the activation is computed from the rounded values
          // while that store reads the tile, and follows through the same tile to d.
#pragma unroll 1
          for (int h = 0; h < NB; ++h) {
            uint32_t keep[2][16];
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              const int c = cgrp * (BLOCK_N / 64) + h * 2 + cc;
              uint32_t r[32];
              tmem_ld_32x32(taddr + c * 32, r);
              if (cc == 0 && store_pending) {
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
                store_pending = false;
              }
              tmem_ld_wait();
              if (h == NB - 1 && cc == 1) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
              }
              const int col0 = n_blk * BLOCK_N + c * 32;
              float v[32];
              if (empty_k) {
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = 0u;
              }
              if (row < M && col0 < N) {
                epilogue_math<false, true>(epu, r, row, col0, N, v);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0.f;
              }
#pragma unroll
              for (int i = 0; i < 16; ++i) keep[cc][i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
#pragma unroll
              for (int qq = 0; qq < 4; ++qq) {
                const uint32_t addr = stg + lane * (SC * 2) + (((cc * 4 + qq) ^ (lane & (CPR - 1))) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(keep[cc][qq * 4 + 0]), "r"(keep[cc][qq * 4 + 1]),
                             "r"(keep[cc][qq * 4 + 2]), "r"(keep[cc][qq * 4 + 3]) : "memory");
              }
            }
            const int colb = n_blk * BLOCK_N + cgrp * (BLOCK_N / 2) + h * SC;
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmAux, stg, colb, static_cast<int>((static_cast<long long>(m_blk) * kBlockM + q * 32)));
              tma_store_commit();
            }
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              const int col0 = colb + cc * 32;
              float v[32];
              uint32_t dummy[32];
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float2 f = unpack_bf16x2(keep[cc][i]);
                v[2 * i] = f.x; v[2 * i + 1] = f.y;
              }
              if (row < M && col0 < N) epilogue_math<false, false, true>(epu, dummy, row, col0, N, v);
#pragma unroll
              for (int i = 0; i < 16; ++i) keep[cc][i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
            }
            if (lane == 0) tma_store_wait_read<0>();       // the pre-activation tile has been read out
            __syncwarp();
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
              for (int qq = 0; qq < 4; ++qq) {
                const uint32_t addr = stg + lane * (SC * 2) + (((cc * 4 + qq) ^ (lane & (CPR - 1))) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(keep[cc][qq * 4 + 0]), "r"(keep[cc][qq * 4 + 1]),
                             "r"(keep[cc][qq * 4 + 2]), "r"(keep[cc][qq * 4 + 3]) : "memory");
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmD, stg, colb, static_cast<int>((static_cast<long long>(m_blk) * kBlockM + q * 32)));
              tma_store_commit();
            }
            store_pending = true;
          }
          continue;
        }
        const int num_pass = two_pass ? 2 : 1;
#pragma unroll 1
        for (int hp = 0; hp < NB * num_pass; ++hp) {
          // with a saved pre-activation every column block is read from TMEM twice: first the pre-activation
          // goes out to aux_out, then the activated value to d
          const int h = hp / num_pass;
          const bool pre_pass = two_pass && (hp - h * num_pass) == 0;
          const bool last_pass = hp == NB * num_pass - 1;
          __nv_bfloat16* dbase = pre_pass ? epu.aux_out : reinterpret_cast<__nv_bfloat16*>(epu.d);
          const long long dld = pre_pass ? epu.ld_aux_out : epu.ldd;
#pragma unroll 1
          for (int cc = 0; cc < SC / 32; ++cc) {
            const int c = cgrp * (BLOCK_N / 64) + h * (SC / 32) + cc;
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            if (cc == 0 && store_pending) {
              // the bulk store issued for the previous block has to be done reading the tile before it is overwritten
              if (lane == 0) tma_store_wait_read<0>();
              __syncwarp();
              store_pending = false;
            }
            tmem_ld_wait();
            if (last_pass && cc == SC / 32 - 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
            }
            const int col0 = n_blk * BLOCK_N + c * 32;
            float v[32];
            if (empty_k) {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = 0u;
            }
            if (row < M && col0 < N) {
              if (pre_pass) epilogue_math<false, true>(epu, r, row, col0, N, v);
              else epilogue_math<false, false>(epu, r, row, col0, N, v);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = 0.f;
            }
#pragma unroll
            for (int qq = 0; qq < 4; ++qq) {
              const int chunk = cc * 4 + qq;
              const uint32_t addr = stg + lane * (SC * 2) + ((chunk ^ (lane & (CPR - 1))) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                           "r"(pack_bf16x2(v[qq * 8 + 0], v[qq * 8 + 1])), "r"(pack_bf16x2(v[qq * 8 + 2], v[qq * 8 + 3])),
                           "r"(pack_bf16x2(v[qq * 8 + 4], v[qq * 8 + 5])), "r"(pack_bf16x2(v[qq * 8 + 6], v[qq * 8 + 7]))
                           : "memory");
            }
          }
          if (SC == 64 && epu.staged == 2) {
            // the tile leaves through a bulk tensor store; rows and columns past the matrix are clipped by the copy
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(pre_pass ? &tmAux : &tmD, stg, n_blk * BLOCK_N + cgrp * (BLOCK_N / 2) + h * SC,
                           static_cast<int>(static_cast<long long>(m_blk) * kBlockM + q * 32));
              tma_store_commit();
            }
            store_pending = true;
            continue;
          }
          __syncwarp();
          constexpr int RPI = 32 / CPR;                            // rows written per warp instruction
          const int ch = lane % CPR, rsub = lane / CPR;
          const int colg = n_blk * BLOCK_N + cgrp * (BLOCK_N / 2) + h * SC + ch * 8;
#pragma unroll 4
          for (int r0 = 0; r0 < 32; r0 += RPI) {
            const int rl = r0 + rsub;
            const long long rg = static_cast<long long>(m_blk) * kBlockM + q * 32 + rl;
            uint4 val;
            const uint32_t addr = stg + rl * (SC * 2) + ((ch ^ (rl & (CPR - 1))) << 4);
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w) : "r"(addr));
            if (rg < M && colg < N) *reinterpret_cast<uint4*>(dbase + rg * dld + colg) = val;
          }
          __syncwarp();
        }
        continue;
      }
#pragma unroll 1
      for (int c = cgrp * (BLOCK_N / 64); c < (cgrp + 1) * (BLOCK_N / 64); ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (empty_k) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (c == (cgrp + 1) * (BLOCK_N / 64) - 1) {
          // all of this warp's accumulator reads are done: hand the buffer back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
        }
        const int col0 = n_blk * BLOCK_N + c * 32;
        if (row < M && col0 < N) epilogue_chunk(epu, r, row, col0, N);
      }
    }
    while (next_item < remote_items && !*abort_flag) copy_one();
    if (lane == 0) tma_store_wait<0>();      // bulk stores of the last tiles have left shared memory and landed
  }

  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      // give copies and MMAs that are still in flight time to land before TMEM is released
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Two-CTA variant (cta_group::2): the two CTAs of a cluster share one 256 x BLOCK_N output tile.  Each CTA loads the
// 128 rows of A it owns and HALF of the B tile (BLOCK_N / 2 rows) into its own shared memory; the even CTA issues
// tcgen05.mma.cta_group::2, which reads both halves of B and writes each CTA's 128 accumulator rows into that CTA's
// TMEM.  Per k-block a CTA moves 16 KB + 16 KB instead of 16 KB + 32 KB through the L2 -> SM fabric, which is what
// bounds the one-CTA kernel on short-K problems.  No TMA multicast: every load targets the loading CTA's own memory
// and reports its bytes to the leader's barrier; tcgen05.commit signals both CTAs' barriers.
// Plain (non-grouped, non-peer) problems only; the epilogue is the staged / direct epilogue of the one-CTA kernel.
// ------------------------------------------------------------------------------------------------------------------
template <int BLOCK_N, int STAGES>
struct SmemLayoutPair {
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = (BLOCK_N / 2) * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 4) * 8 + 16;
  static constexpr int kStageCols = (BLOCK_N % 128 == 0) ? 64 : 32;
  static constexpr int kStagingOffset = (kTotal + 1023) & ~1023;   // 1024-byte aligned: the tiles are also TMA-store sources (128B swizzle)
  static constexpr int kStagingBytesPerWarp = 32 * kStageCols * 2;
  static constexpr int kTotalStaged = kStagingOffset + kNumEpilogueWarps * kStagingBytesPerWarp;
};

template <int A_MN, int B_MN, int BLOCK_N, int STAGES, int FP8 = 0>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmAux, int M, int N,
                      int K, int group_m, int num_splits, int kb_per_split, long long d_split_stride, EpiParams ep,
                      unsigned int* status) {
  using L = SmemLayoutPair<BLOCK_N, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = smem_u32(bars + STAGES);
  const uint32_t bar_tfull = smem_u32(bars + 2 * STAGES);
  const uint32_t bar_tempty = smem_u32(bars + 2 * STAGES + 2);
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();       // 0: leader (issues the MMAs), 1: peer
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  constexpr uint32_t kTmemCols = (2 * BLOCK_N <= 64) ? 64 : (2 * BLOCK_N <= 128) ? 128 : (2 * BLOCK_N <= 256) ? 256 : 512;
  constexpr int kPairM = 2 * kBlockM;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);                // leader: its own expect_tx arrival (+ both CTAs' bytes)
      mbar_init(bar_empty + 8 * s, 1);               // one multicast commit per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 2 * kNumEpilogueWarps);   // leader: the epilogue warps of both CTAs
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_ptr_smem), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                 // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int num_m = (M + kPairM - 1) / kPairM;
  const int num_n = (N + BLOCK_N - 1) / BLOCK_N;
  const int num_tiles = num_m * num_n;
  const int num_kb_total = (K + kBlockK - 1) / kBlockK;
  const int group_size = group_m * num_n;
  const int num_units = num_tiles * num_splits;

  auto decode_tile = [&](int unit, int& m_blk, int& n_blk, int& kb0, int& kb1, int& split) {
    split = unit / num_tiles;
    const int tile = unit - split * num_tiles;
    kb0 = split * kb_per_split;
    kb1 = min(num_kb_total, kb0 + kb_per_split);
    const int group = tile / group_size;
    const int first_m = group * group_m;
    const int gm = min(group_m, num_m - first_m);
    const int in_group = tile - group * group_size;
    m_blk = first_m + in_group % gm;
    n_blk = in_group / gm;
  };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer (both CTAs)
      uint32_t it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_units && ok; tile += num_clusters) {
        int m_blk, n_blk, kb0, kb1, split;
        decode_tile(tile, m_blk, n_blk, kb0, kb1, split);
        const int a_row = m_blk * kPairM + static_cast<int>(cta_rank) * kBlockM;
        const int b_row = n_blk * BLOCK_N + static_cast<int>(cta_rank) * (BLOCK_N / 2);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, status, 11)) { ok = false; break; }
          const uint32_t full_local = bar_full + 8 * s;
          if (cta_rank == 0) mbar_arrive_expect_tx(full_local, 2 * L::kStageBytes);
          const uint32_t full = mapa_shared(full_local, 0);
          const uint32_t sa = smem_base + s * L::kStageBytes;
          const uint32_t sb = sa + L::kABytes;
          if (A_MN == 0) {
            tma_load_2d_pair(sa, &tmA, kb * kBlockK * (FP8 ? 2 : 1), a_row, full);
          } else {
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j)
              tma_load_2d_pair(sa + j * (kBlockK * 128), &tmA, a_row + j * 64, kb * kBlockK, full);
          }
          if (B_MN == 0) {
            tma_load_2d_pair(sb, &tmB, kb * kBlockK * (FP8 ? 2 : 1), b_row, full);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_N / 2 / 64; ++j)
              tma_load_2d_pair(sb + j * (kBlockK * 128), &tmB, b_row + j * 64, kb * kBlockK, full);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && cta_rank == 0) {
      // ------------------------------------------------------------------ MMA issuer (leader CTA only)
      const uint32_t idesc = FP8 ? (umma_idesc_e4m3(kPairM, BLOCK_N) | (static_cast<uint32_t>(ep.fp8_b_format) << 10))
                                 : umma_idesc_bf16(kPairM, BLOCK_N, A_MN, B_MN);
      uint32_t it = 0, t = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_units && ok; tile += num_clusters, ++t) {
        int m_blk, n_blk, kb0, kb1, split;
        decode_tile(tile, m_blk, n_blk, kb0, kb1, split);
        const uint32_t acc = t & 1, acc_ph = (t >> 1) & 1;
        if (!mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, abort_flag, status, 12)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BLOCK_N;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, status, 13)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + s * L::kStageBytes;
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t da = A_MN ? umma_smem_desc_sw128(sa + k * (kUmmaK * 128), kBlockK * 128, 1024)
                                     : umma_smem_desc_sw128(sa + k * (kUmmaK * 2), 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc_sw128(sb + k * (kUmmaK * 128), kBlockK * 128, 1024)
                                     : umma_smem_desc_sw128(sb + k * (kUmmaK * 2), 16, 1024);
            if (FP8) umma_f8_ss_pair(tmem_d, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
            else umma_bf16_ss_pair(tmem_d, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit_pair(bar_empty + 8 * s, 3);     // both CTAs may refill this stage
        }
        if (ok) umma_commit_pair(bar_tfull + 8 * acc, 3);   // both CTAs' accumulator halves are complete
      }
    }
  } else {
    // -------------------------------------------------------------------- epilogue warps (both CTAs)
    const int q = warp & 3;
    const int ew = warp - 2;
    const int cgrp = ew >> 2;
    bool store_pending = false;
    uint32_t t = 0;
    for (int tile = cluster_id; tile < num_units; tile += num_clusters, ++t) {
      int m_blk, n_blk, kb0, kb1, split;
      decode_tile(tile, m_blk, n_blk, kb0, kb1, split);
      EpiParams epu = ep;
      if (num_splits > 1)
        epu.d = reinterpret_cast<float*>(ep.d) + static_cast<long long>(split) * d_split_stride;
      const uint32_t acc = t & 1, acc_ph = (t >> 1) & 1;
      if (!mbar_wait(bar_tfull + 8 * acc, acc_ph, abort_flag, status, 14)) break;
      tc_fence_after();
      const long long row0 = static_cast<long long>(m_blk) * kPairM + static_cast<long long>(cta_rank) * kBlockM + q * 32;
      const long long row = row0 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BLOCK_N;
      const uint32_t tempty_leader = mapa_shared(bar_tempty + 8 * acc, 0);
      if (epu.staged) {
        constexpr int SC = L::kStageCols, CPR = SC / 8;
        const uint32_t stg = smem_base + L::kStagingOffset + ew * L::kStagingBytesPerWarp;
        constexpr int NB = (BLOCK_N / 2) / SC;
        const bool two_pass = epu.aux_out != nullptr &&
                              (epu.act == RB_ACT_GELU || epu.act == RB_ACT_RELU || epu.act == RB_ACT_SILU);
        if (SC == 64 && epu.staged == 2 && two_pass) {
          // One pass over the accumulator: the pre-activation is rounded to bf16, kept packed in registers for the 64
          // columns of a block and sent to aux_out by a bulk store; the activation is computed from the rounded values
          // while that store reads the tile, and follows through the same tile to d.
#pragma unroll 1
          for (int h = 0; h < NB; ++h) {
            uint32_t keep[2][16];
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              const int c = cgrp * (BLOCK_N / 64) + h * 2 + cc;
              uint32_t r[32];
              tmem_ld_32x32(taddr + c * 32, r);
              if (cc == 0 && store_pending) {
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
                store_pending = false;
              }
              tmem_ld_wait();
              if (h == NB - 1 && cc == 1) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(tempty_leader);
              }
              const int col0 = n_blk * BLOCK_N + c * 32;
              float v[32];
              if (false) {
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = 0u;
              }
              if (row < M && col0 < N) {
                epilogue_math<false, true>(epu, r, row, col0, N, v);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0.f;
              }
#pragma unroll
              for (int i = 0; i < 16; ++i) keep[cc][i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
#pragma unroll
              for (int qq = 0; qq < 4; ++qq) {
                const uint32_t addr = stg + lane * (SC * 2) + (((cc * 4 + qq) ^ (lane & (CPR - 1))) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(keep[cc][qq * 4 + 0]), "r"(keep[cc][qq * 4 + 1]),
                             "r"(keep[cc][qq * 4 + 2]), "r"(keep[cc][qq * 4 + 3]) : "memory");
              }
            }
            const int colb = n_blk * BLOCK_N + cgrp * (BLOCK_N / 2) + h * SC;
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmAux, stg, colb, static_cast<int>(row0));
              tma_store_commit();
            }
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              const int col0 = colb + cc * 32;
              float v[32];
              uint32_t dummy[32];
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float2 f = unpack_bf16x2(keep[cc][i]);
                v[2 * i] = f.x; v[2 * i + 1] = f.y;
              }
              if (row < M && col0 < N) epilogue_math<false, false, true>(epu, dummy, row, col0, N, v);
#pragma unroll
              for (int i = 0; i < 16; ++i) keep[cc][i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
            }
            if (lane == 0) tma_store_wait_read<0>();       // the pre-activation tile has been read out
            __syncwarp();
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
              for (int qq = 0; qq < 4; ++qq) {
                const uint32_t addr = stg + lane * (SC * 2) + (((cc * 4 + qq) ^ (lane & (CPR - 1))) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(keep[cc][qq * 4 + 0]), "r"(keep[cc][qq * 4 + 1]),
                             "r"(keep[cc][qq * 4 + 2]), "r"(keep[cc][qq * 4 + 3]) : "memory");
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmD, stg, colb, static_cast<int>(row0));
              tma_store_commit();
            }
            store_pending = true;
          }
          continue;
        }
        const int num_pass = two_pass ? 2 : 1;
#pragma unroll 1
        for (int hp = 0; hp < NB * num_pass; ++hp) {
          const int h = hp / num_pass;
          const bool pre_pass = two_pass && (hp - h * num_pass) == 0;
          const bool last_pass = hp == NB * num_pass - 1;
          __nv_bfloat16* dbase = pre_pass ? epu.aux_out : reinterpret_cast<__nv_bfloat16*>(epu.d);
          const long long dld = pre_pass ? epu.ld_aux_out : epu.ldd;
#pragma unroll 1
          for (int cc = 0; cc < SC / 32; ++cc) {
            const int c = cgrp * (BLOCK_N / 64) + h * (SC / 32) + cc;
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            if (cc == 0 && store_pending) {
              // the bulk store issued for the previous block has to be done reading the tile before it is overwritten
              if (lane == 0) tma_store_wait_read<0>();
              __syncwarp();
              store_pending = false;
            }
            tmem_ld_wait();
            if (last_pass && cc == SC / 32 - 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(tempty_leader);
            }
            const int col0 = n_blk * BLOCK_N + c * 32;
            float v[32];
            if (row < M && col0 < N) {
              if (pre_pass) epilogue_math<false, true>(epu, r, row, col0, N, v);
              else epilogue_math<false, false>(epu, r, row, col0, N, v);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = 0.f;
            }
#pragma unroll
            for (int qq = 0; qq < 4; ++qq) {
              const int chunk = cc * 4 + qq;
              const uint32_t addr = stg + lane * (SC * 2) + ((chunk ^ (lane & (CPR - 1))) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                           "r"(pack_bf16x2(v[qq * 8 + 0], v[qq * 8 + 1])), "r"(pack_bf16x2(v[qq * 8 + 2], v[qq * 8 + 3])),
                           "r"(pack_bf16x2(v[qq * 8 + 4], v[qq * 8 + 5])), "r"(pack_bf16x2(v[qq * 8 + 6], v[qq * 8 + 7]))
                           : "memory");
            }
          }
          if (SC == 64 && epu.staged == 2) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(pre_pass ? &tmAux : &tmD, stg, n_blk * BLOCK_N + cgrp * (BLOCK_N / 2) + h * SC, static_cast<int>(row0));
              tma_store_commit();
            }
            store_pending = true;
            continue;
          }
          __syncwarp();
          constexpr int RPI = 32 / CPR;
          const int ch = lane % CPR, rsub = lane / CPR;
          const int colg = n_blk * BLOCK_N + cgrp * (BLOCK_N / 2) + h * SC + ch * 8;
#pragma unroll 4
          for (int r0 = 0; r0 < 32; r0 += RPI) {
            const int rl = r0 + rsub;
            const long long rg = row0 + rl;
            uint4 val;
            const uint32_t addr = stg + rl * (SC * 2) + ((ch ^ (rl & (CPR - 1))) << 4);
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w) : "r"(addr));
            if (rg < M && colg < N) *reinterpret_cast<uint4*>(dbase + rg * dld + colg) = val;
          }
          __syncwarp();
        }
        continue;
      }
#pragma unroll 1
      for (int c = cgrp * (BLOCK_N / 64); c < (cgrp + 1) * (BLOCK_N / 64); ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (c == (cgrp + 1) * (BLOCK_N / 64) - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tempty_leader);
        }
        const int col0 = n_blk * BLOCK_N + c * 32;
        if (row < M && col0 < N) epilogue_chunk(epu, r, row, col0, N);
      }
    }
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                 // the leader's MMAs read this CTA's shared memory until here
  if (warp == 1) {
    if (*abort_flag) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// d (+)= sum_s ws[s] (+ bias) (+ residual)  (slabs of M*N fp32, dense), s ascending: the order is fixed, so the
// result is reproducible.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, int splits, long long slab, void* d, long long ldd, int M, int N,
                     int out_f32, int accumulate, const __nv_bfloat16* __restrict__ bias,
                     const __nv_bfloat16* __restrict__ residual, long long ldr) {
  const long long n4 = static_cast<long long>(M) * N / 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 acc = reinterpret_cast<const float4*>(ws)[i];
    for (int s = 1; s < splits; ++s) {
      const float4 v = reinterpret_cast<const float4*>(ws + s * slab)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const long long e = i * 4;
    const long long row = e / N;
    const int col = static_cast<int>(e - row * N);
    if (bias != nullptr) {
      const uint2 b = __ldg(reinterpret_cast<const uint2*>(bias + col));
      const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y);
      acc.x += b0.x; acc.y += b0.y; acc.z += b1.x; acc.w += b1.y;
    }
    if (residual != nullptr) {
      const uint2 r = __ldg(reinterpret_cast<const uint2*>(residual + row * ldr + col));
      const float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y);
      acc.x += r0.x; acc.y += r0.y; acc.z += r1.x; acc.w += r1.y;
    }
    if (out_f32) {
      float4* dp = reinterpret_cast<float4*>(reinterpret_cast<float*>(d) + row * ldd + col);
      if (accumulate) { const float4 o = *dp; acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w; }
      *dp = acc;
    } else {
      uint2* dp = reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(d) + row * ldd + col);
      if (accumulate) {
        const uint2 o = *dp;
        const float2 a = unpack_bf16x2(o.x), b = unpack_bf16x2(o.y);
        acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
      }
      uint2 o;
      o.x = pack_bf16x2(acc.x, acc.y);
      o.y = pack_bf16x2(acc.z, acc.w);
      *dp = o;
    }
  }
}

}  // namespace rb

// ---------------------------------------------------------------------------------------------
// host launcher
// ---------------------------------------------------------------------------------------------
namespace {

// RUSTRAL_GEMM_STAGED=0/1 turns the shared-memory staged output path off / on for ordinary (non-peer) GEMMs.
bool staged_store_default() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("RUSTRAL_GEMM_STAGED");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// Staged 64-column tiles leave through bulk tensor stores (one instruction per tile instead of eight ld.shared /
// st.global pairs per thread); RUSTRAL_GEMM_TMA_STORE=0 keeps the load / store loop.  Measured on one B200, same process:
// bias + GELU + saved pre-activation 32768 x 3072 x 768 224 -> 194 us, QKV shape 99.3 -> 95.3 us, 8192^3 unchanged.
bool tma_store_default() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("RUSTRAL_GEMM_TMA_STORE");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <int A_MN, int B_MN, int BLOCK_N, int STAGES, int FP8 = 0>
int launch(const RbGemmArgs& g, const CUtensorMap* ta, const CUtensorMap* tb, int grid, int splits, cudaStream_t stream) {
  using L = rb::SmemLayout<BLOCK_N, STAGES>;
  const CUtensorMap* td = ta;        // placeholders unless the bulk-store epilogue is chosen below
  const CUtensorMap* tx = ta;
  auto kern = rb::gemm_bf16_kernel<A_MN, B_MN, BLOCK_N, STAGES, FP8>;
  // Staged (coalesced) stores: plain bf16 outputs whose rows are whole 16-byte chunks.  Always on for peer stores.
  const bool can_stage = !g.out_f32 && !g.accumulate && splits <= 1 && (g.N % 8 == 0) && g.group_mode != 2 &&
                         L::kTotalStaged + 1024 <= 232448;
  const bool staged = can_stage && (g.peer_mode == 2 || staged_store_default());
  if (g.peer_mode == 2 && !staged) return -11;
  const int smem = (staged ? L::kTotalStaged : L::kTotal) + 1024;
  static int configured_dev[64] = {0};   // per instantiation and device: largest size set so far
  int& configured = configured_dev[rbhost::device_slot()];
  if (configured < smem) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = smem;
  }
  rb::EpiParams ep;
  ep.d = g.d; ep.ldd = g.ldd;
  ep.bias = reinterpret_cast<const __nv_bfloat16*>(g.bias);
  ep.residual = reinterpret_cast<const __nv_bfloat16*>(g.residual); ep.ldr = g.ldr;
  ep.aux_in = reinterpret_cast<const __nv_bfloat16*>(g.aux_in); ep.ld_aux_in = g.ld_aux_in;
  ep.aux_out = reinterpret_cast<__nv_bfloat16*>(g.aux_out); ep.ld_aux_out = g.ld_aux_out;
  ep.act = g.act; ep.out_f32 = g.out_f32; ep.accumulate = g.accumulate; ep.alpha = g.alpha;
  ep.staged = staged ? 1 : 0;
  if (staged && g.peer_mode == 0 && L::kStageCols == 64 && tma_store_default()) {
    int err = 0;
    td = rbhost::get_tmap_2d(g.d, 2, (uint64_t)g.N, (uint64_t)g.M, (uint64_t)g.ldd, 64, 32, 1, &err);
    tx = g.aux_out ? rbhost::get_tmap_2d(g.aux_out, 2, (uint64_t)g.N, (uint64_t)g.M, (uint64_t)g.ld_aux_out, 64, 32, 1, &err) : td;
    if (td && tx) ep.staged = 2;
    else { td = ta; tx = ta; }
  }
  ep.row_scale = reinterpret_cast<const float*>(g.a_scale);
  ep.col_scale = reinterpret_cast<const float*>(g.b_scale);
  ep.fp8_b_format = g.ab_fp8 == 2 ? 1 : 0;
  const int group_m = g.group_m > 0 ? g.group_m : 8;
  const int k_units = FP8 ? (g.K + 1) / 2 : g.K;          // the kernel counts K in two-byte units
  const int num_kb = (k_units + rb::kBlockK - 1) / rb::kBlockK;
  int kb_per = num_kb;
  long long slab = 0;
  if (splits > 1) {
    kb_per = (num_kb + splits - 1) / splits;
    splits = (num_kb + kb_per - 1) / kb_per;   // no split may end up with an empty K range
    slab = static_cast<long long>(g.M) * g.N;
    ep.d = g.workspace; ep.ldd = g.N; ep.out_f32 = 1; ep.accumulate = 0;
    ep.bias = nullptr; ep.residual = nullptr;          // applied once, by the kernel that folds the slabs
  }
  rb::GroupInfo grp;
  grp.mode = g.group_mode; grp.num_experts = g.num_experts;
  grp.tile_expert = reinterpret_cast<const int*>(g.tile_expert);
  grp.num_m_tiles = reinterpret_cast<const int*>(g.num_m_tiles);
  grp.offsets = reinterpret_cast<const int*>(g.expert_offsets);
  grp.b_expert_rows = g.b_expert_rows; grp.d_expert_stride = g.d_expert_stride;
  grp.tile_arrived = reinterpret_cast<const unsigned int*>(g.tile_arrived);
  grp.tile_expected = reinterpret_cast<const int*>(g.tile_expected);
  rb::PeerInfo peer;
  memset(&peer, 0, sizeof(peer));
  peer.mode = g.peer_mode; peer.world = g.peer_world; peer.rank = g.peer_rank; peer.rows_per_rank = g.rows_per_rank;
  peer.a_full = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(g.peer_mode == 3 ? g.b : g.a));
  peer.ready = reinterpret_cast<unsigned int*>(g.ready_flags);
  peer.epoch = g.peer_epoch;
  for (int r = 0; r < 8; ++r) {
    peer.a_peer[r] = reinterpret_cast<const __nv_bfloat16*>(g.peer_ptrs[r]);
    peer.d_peer[r] = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(g.peer_ptrs[r]));
  }
  kern<<<grid, rb::kNumThreads, smem, stream>>>(*ta, *tb, *td, *tx, g.M, g.N, k_units, group_m, splits, kb_per, slab, ep, grp, peer,
                                                rbhost::status_ptr());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || splits <= 1) return static_cast<int>(e);
  const long long n4 = slab / 4;
  int rgrid = static_cast<int>((n4 + 255) / 256 < 148 * 8 ? (n4 + 255) / 256 : 148 * 8);
  rb::splitk_reduce_kernel<<<rgrid, 256, 0, stream>>>(reinterpret_cast<const float*>(g.workspace), splits, slab, g.d,
                                                      g.ldd, g.M, g.N, g.out_f32, g.accumulate,
                                                      reinterpret_cast<const __nv_bfloat16*>(g.bias),
                                                      reinterpret_cast<const __nv_bfloat16*>(g.residual), g.ldr);
  return static_cast<int>(cudaGetLastError());
}

template <int BLOCK_N, int STAGES>
int dispatch_major(const RbGemmArgs& g, const CUtensorMap* ta, const CUtensorMap* tb, int grid, int splits,
                   cudaStream_t s) {
  if (!g.a_mn_major && !g.b_mn_major) return launch<0, 0, BLOCK_N, STAGES>(g, ta, tb, grid, splits, s);
  if (!g.a_mn_major && g.b_mn_major) return launch<0, 1, BLOCK_N, STAGES>(g, ta, tb, grid, splits, s);
  if (g.a_mn_major && g.b_mn_major) return launch<1, 1, BLOCK_N, STAGES>(g, ta, tb, grid, splits, s);
  return launch<1, 0, BLOCK_N, STAGES>(g, ta, tb, grid, splits, s);
}

// RUSTRAL_GEMM_2CTA=0 keeps every problem on the one-CTA kernel.
bool pair_kernel_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("RUSTRAL_GEMM_2CTA");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <int A_MN, int B_MN, int FP8 = 0>
int launch_pair(const RbGemmArgs& g, const CUtensorMap* ta, const CUtensorMap* tb_half, int clusters, int splits,
                cudaStream_t stream) {
  constexpr int BLOCK_N = 256, STAGES = 6;
  using L = rb::SmemLayoutPair<BLOCK_N, STAGES>;
  auto kern = rb::gemm_bf16_pair_kernel<A_MN, B_MN, BLOCK_N, STAGES, FP8>;
  const bool staged = !g.out_f32 && !g.accumulate && splits <= 1 && (g.N % 8 == 0) && staged_store_default() &&
                      L::kTotalStaged + 1024 <= 232448;
  const int smem = (staged ? L::kTotalStaged : L::kTotal) + 1024;
  static int configured_dev[64] = {0};
  int& configured = configured_dev[rbhost::device_slot()];
  if (configured < smem) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = smem;
  }
  rb::EpiParams ep;
  ep.d = g.d; ep.ldd = g.ldd;
  ep.bias = reinterpret_cast<const __nv_bfloat16*>(g.bias);
  ep.residual = reinterpret_cast<const __nv_bfloat16*>(g.residual); ep.ldr = g.ldr;
  ep.aux_in = reinterpret_cast<const __nv_bfloat16*>(g.aux_in); ep.ld_aux_in = g.ld_aux_in;
  ep.aux_out = reinterpret_cast<__nv_bfloat16*>(g.aux_out); ep.ld_aux_out = g.ld_aux_out;
  ep.act = g.act; ep.out_f32 = g.out_f32; ep.accumulate = g.accumulate; ep.alpha = g.alpha;
  ep.staged = staged ? 1 : 0;
  const CUtensorMap* td = ta;
  const CUtensorMap* tx = ta;
  if (staged && tma_store_default()) {
    int err = 0;
    td = rbhost::get_tmap_2d(g.d, 2, (uint64_t)g.N, (uint64_t)g.M, (uint64_t)g.ldd, 64, 32, 1, &err);
    tx = g.aux_out ? rbhost::get_tmap_2d(g.aux_out, 2, (uint64_t)g.N, (uint64_t)g.M, (uint64_t)g.ld_aux_out, 64, 32, 1, &err) : td;
    if (td && tx) ep.staged = 2;
    else { td = ta; tx = ta; }
  }
  ep.row_scale = reinterpret_cast<const float*>(g.a_scale);
  ep.col_scale = reinterpret_cast<const float*>(g.b_scale);
  ep.fp8_b_format = g.ab_fp8 == 2 ? 1 : 0;
  const int group_m = g.group_m > 0 ? g.group_m : 4;      // in 256-row units
  const int k_units = FP8 ? (g.K + 1) / 2 : g.K;
  const int num_kb = (k_units + rb::kBlockK - 1) / rb::kBlockK;
  int kb_per = num_kb;
  long long slab = 0;
  if (splits > 1) {
    kb_per = (num_kb + splits - 1) / splits;
    splits = (num_kb + kb_per - 1) / kb_per;
    slab = static_cast<long long>(g.M) * g.N;
    ep.d = g.workspace; ep.ldd = g.N; ep.out_f32 = 1; ep.accumulate = 0;
    ep.bias = nullptr; ep.residual = nullptr;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(rb::kNumThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, *ta, *tb_half, *td, *tx, g.M, g.N, k_units, group_m, splits, kb_per, slab, ep,
                                     rbhost::status_ptr());
  if (e != cudaSuccess || splits <= 1) return static_cast<int>(e);
  const long long n4 = slab / 4;
  int rgrid = static_cast<int>((n4 + 255) / 256 < 148 * 8 ? (n4 + 255) / 256 : 148 * 8);
  rb::splitk_reduce_kernel<<<rgrid, 256, 0, stream>>>(reinterpret_cast<const float*>(g.workspace), splits, slab, g.d,
                                                      g.ldd, g.M, g.N, g.out_f32, g.accumulate,
                                                      reinterpret_cast<const __nv_bfloat16*>(g.bias),
                                                      reinterpret_cast<const __nv_bfloat16*>(g.residual), g.ldr);
  return static_cast<int>(cudaGetLastError());
}

// Relative time of one tile column unit per tile width: narrow tiles re-read the A operand from shared
// memory more often per MMA (measured on B200: 128-wide runs ~1.3x, 64-wide ~2.3x slower than 256-wide).
int width_cost(int bn) { return bn == 256 ? 100 : bn == 192 ? 104 : bn == 128 ? 132 : 235; }

long long plan_cost(int M, int N, int bn, int splits, int sms, bool pair_ok) {
  const long long tiles = static_cast<long long>((M + 127) / 128) * ((N + bn - 1) / bn) * splits;
  const long long waves = (tiles + sms - 1) / sms;
  // 256-wide plans of plain problems run on the two-CTA kernel, measured about 10 % faster per tile
  const int wc = (bn == 256 && pair_ok) ? 88 : width_cost(bn);
  // per-unit time ~ bn * K/splits (+ a fixed prologue/epilogue share that split-K multiplies)
  return waves * bn * wc * (1000 / splits + 40);
}

void pick_plan(const RbGemmArgs& g, int sms, int& bn_out, int& splits_out) {
  const int cands[4] = {256, 192, 128, 64};
  const int split_cands[7] = {1, 2, 3, 4, 6, 8, 12};
  const bool can_split = g.group_mode == 0 && g.peer_mode == 0 && g.workspace != nullptr && g.act == RB_ACT_NONE && !g.aux_out &&
                         !g.a_scale && !g.b_scale && !g.ab_fp8 &&
                         (g.N % 4 == 0) && (static_cast<long long>(g.M) * g.N % 4 == 0) && (!g.residual || (g.ldr % 4 == 0));
  const bool pair_ok = g.peer_mode == 0 && g.group_mode == 0 && g.M > 128 && g.max_ctas == 0 && pair_kernel_enabled();
  long long best = -1;
  bn_out = 128; splits_out = 1;
  for (int c = 0; c < 4; ++c) {
    const int bn = cands[c];
    if (g.block_n && g.block_n != bn) continue;
    if (!g.block_n && bn > 64 && g.N <= bn / 2) continue;
    for (int si = 0; si < 7; ++si) {
      const int sp = split_cands[si];
      if (g.splits > 0 && sp != g.splits) continue;
      if (sp > 1) {
        if (!can_split) continue;
        if (g.splits <= 0 && g.K / sp < 1024) continue;
        if (static_cast<long long>(sp) * g.M * g.N * 4 > g.workspace_bytes) continue;
      }
      const long long cost = plan_cost(g.M, g.N, bn, sp, sms, pair_ok);
      if (best < 0 || cost < best) { best = cost; bn_out = bn; splits_out = sp; }
    }
  }
}

// 8-bit floating-point operands: byte tensor maps with 128-element boxes, K-major only.
int gemm_fp8(const RbGemmArgs& g, int sms, int bn, int splits, cudaStream_t stream) {
  if (g.a_mn_major || g.b_mn_major || g.peer_mode != 0 || g.group_mode == 2) return -12;
  if ((g.lda & 15) || (g.ldb & 15) || (g.K & 15)) return -2;
  int err = 0;
  const CUtensorMap* ta = rbhost::get_tmap_2d(g.a, 1, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, 128, 128, 1, &err);
  if (!ta) return err ? err : -5;
  const uint64_t b_experts = g.group_mode == 1 ? (uint64_t)g.num_experts : 1;
  if (bn == 256 && g.group_mode == 0 && g.M > 128 && g.max_ctas == 0 && pair_kernel_enabled()) {
    const CUtensorMap* tb_half = rbhost::get_tmap_2d(g.b, 1, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, 128, 128, 1, &err);
    if (!tb_half) return err ? err : -5;
    const long long tiles2 = (long long)((g.M + 255) / 256) * ((g.N + 255) / 256) * splits;
    const int max_clusters = sms / 2;
    const int clusters = static_cast<int>(tiles2 < max_clusters ? tiles2 : max_clusters);
    return launch_pair<0, 0, 1>(g, ta, tb_half, clusters, splits, stream);
  }
  const CUtensorMap* tb = rbhost::get_tmap_2d(g.b, 1, (uint64_t)g.K, (uint64_t)g.N * b_experts, (uint64_t)g.ldb, 128, (uint32_t)bn, 1, &err);
  if (!tb) return err ? err : -5;
  const long long tiles = (long long)((g.M + 127) / 128) * ((g.N + bn - 1) / bn) * splits;
  int grid = static_cast<int>(tiles < sms ? tiles : sms);
  if (g.max_ctas > 0 && grid > g.max_ctas) grid = g.max_ctas;
  switch (bn) {
    case 256: return launch<0, 0, 256, 4, 1>(g, ta, tb, grid, splits, stream);
    case 192: return launch<0, 0, 192, 5, 1>(g, ta, tb, grid, splits, stream);
    case 128: return launch<0, 0, 128, 6, 1>(g, ta, tb, grid, splits, stream);
    default: return launch<0, 0, 64, 8, 1>(g, ta, tb, grid, splits, stream);
  }
}

}  // namespace

RB_API int rb_gemm_bf16(const RbGemmArgs* args, void* stream_v) {
  const RbGemmArgs& g = *args;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return -1;
  // TMA needs 16-byte aligned bases and pitches
  if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.b) & 15)) return -2;
  if (!g.ab_fp8 && ((g.lda & 7) || (g.ldb & 7))) return -2;
  // vector epilogue accesses need 16-byte aligned rows
  const int dalign = g.out_f32 ? 4 : 8;
  if ((g.ldd % dalign) || (reinterpret_cast<uintptr_t>(g.d) & 15)) return -3;
  if (g.residual && ((g.ldr & 7) || (reinterpret_cast<uintptr_t>(g.residual) & 15))) return -3;
  if (g.aux_in && ((g.ld_aux_in & 7) || (reinterpret_cast<uintptr_t>(g.aux_in) & 15))) return -3;
  if (g.aux_out && ((g.ld_aux_out & 7) || (reinterpret_cast<uintptr_t>(g.aux_out) & 15))) return -3;
  if (g.bias && (reinterpret_cast<uintptr_t>(g.bias) & 15)) return -3;
  if (g.a_scale && (reinterpret_cast<uintptr_t>(g.a_scale) & 3)) return -3;
  if (g.b_scale && (reinterpret_cast<uintptr_t>(g.b_scale) & 15)) return -3;
  if ((g.act >= RB_ACT_DGELU && g.act <= RB_ACT_MUL) && !g.aux_in) return -4;

  if (g.group_mode < 0 || g.group_mode > 2) return -8;
  if (g.group_mode == 1 && (!g.tile_expert || !g.num_m_tiles || g.b_expert_rows <= 0)) return -8;
  if ((g.tile_arrived == nullptr) != (g.tile_expected == nullptr) || (g.tile_arrived && g.group_mode != 1)) return -8;
  if (g.group_mode == 1 && g.b_mn_major && (g.K % 64)) return -8;     // expert K ranges must be whole k-blocks
  if (g.group_mode == 2 && (!g.expert_offsets || g.num_experts <= 0 || !g.a_mn_major || !g.b_mn_major)) return -8;
  if (g.peer_mode < 0 || g.peer_mode > 3) return -11;
  RbGemmArgs forced;
  if (g.peer_mode == 3) {
    // tiles must not straddle two ranks' blocks of B: the tile width divides the rows per rank
    if (g.rows_per_rank <= 0 || (g.rows_per_rank % 128)) return -11;
    const int want = (g.rows_per_rank % 256 == 0) ? 256 : 128;
    if (g.block_n != 0 && g.block_n != 128 && g.block_n != want) return -11;
    if (g.block_n == 0) {
      forced = g;
      forced.block_n = want;
      return rb_gemm_bf16(&forced, stream_v);
    }
  }
  if (g.peer_mode != 0) {
    if (g.peer_world < 2 || g.peer_world > 8 || g.peer_rank < 0 || g.peer_rank >= g.peer_world) return -11;
    if (g.rows_per_rank <= 0 || (g.rows_per_rank % 128) ||
        g.rows_per_rank * g.peer_world != (g.peer_mode == 3 ? g.N : g.M))
      return -11;
    if (g.peer_mode == 3 && (g.b_mn_major || !g.ready_flags || g.ldb != g.K)) return -11;   // b_full is dense [N, K]
    if ((g.peer_mode == 1 && g.a_mn_major) || g.group_mode != 0 || g.out_f32) return -11;
    for (int r = 0; r < g.peer_world; ++r)
      if (!g.peer_ptrs[r] || (reinterpret_cast<uintptr_t>(g.peer_ptrs[r]) & 15)) return -11;
    if (g.peer_mode == 1 && (!g.ready_flags || g.lda != g.K)) return -11;       // a_full is dense [M, K]
  }
  const int sms = rbhost::device_sm_count();
  if (g.block_n != 0 && g.block_n != 64 && g.block_n != 128 && g.block_n != 192 && g.block_n != 256) return -6;
  int bn = 128, splits = 1;
  pick_plan(g, sms, bn, splits);
  if (g.splits > 1 && splits != g.splits) return -7;   // a forced split count that cannot be honoured

  if (g.ab_fp8) return gemm_fp8(g, sms, bn, splits, stream);

  int err = 0;
  const CUtensorMap* ta = g.a_mn_major
                              ? rbhost::get_tmap_2d(g.a, 2, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, 64, 64, 1, &err)
                              : rbhost::get_tmap_2d(g.a, 2, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, 64, 128, 1, &err);
  if (!ta) return err ? err : -5;
  const uint64_t b_experts = g.group_mode == 1 ? (uint64_t)g.num_experts : 1;
  const CUtensorMap* tb = g.b_mn_major
                              ? rbhost::get_tmap_2d(g.b, 2, (uint64_t)g.N, (uint64_t)g.K * b_experts, (uint64_t)g.ldb, 64, 64, 1, &err)
                              : rbhost::get_tmap_2d(g.b, 2, (uint64_t)g.K, (uint64_t)g.N * b_experts, (uint64_t)g.ldb, 64, (uint32_t)bn, 1, &err);
  if (!tb) return err ? err : -5;

  if (bn == 256 && g.peer_mode == 0 && g.group_mode == 0 && g.M > 128 && g.max_ctas == 0 && pair_kernel_enabled()) {
    // two-CTA kernel: 256 x 256 tiles per CTA pair, each CTA loads half of the B tile
    const CUtensorMap* tb_half =
        g.b_mn_major ? tb : rbhost::get_tmap_2d(g.b, 2, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, 64, 128, 1, &err);
    if (!tb_half) return err ? err : -5;
    const long long tiles2 = (long long)((g.M + 255) / 256) * ((g.N + 255) / 256) * splits;
    const int max_clusters = sms / 2;
    const int clusters = static_cast<int>(tiles2 < max_clusters ? tiles2 : max_clusters);
    if (!g.a_mn_major && !g.b_mn_major) return launch_pair<0, 0>(g, ta, tb_half, clusters, splits, stream);
    if (!g.a_mn_major && g.b_mn_major) return launch_pair<0, 1>(g, ta, tb_half, clusters, splits, stream);
    if (g.a_mn_major && g.b_mn_major) return launch_pair<1, 1>(g, ta, tb_half, clusters, splits, stream);
    return launch_pair<1, 0>(g, ta, tb_half, clusters, splits, stream);
  }
  long long tiles = (long long)((g.M + 127) / 128) * ((g.N + bn - 1) / bn) * splits;
  if (g.group_mode == 2) tiles *= g.num_experts;
  int grid = static_cast<int>(tiles < sms ? tiles : sms);
  if (g.max_ctas > 0 && grid > g.max_ctas) grid = g.max_ctas;
  switch (bn) {
    case 256: return dispatch_major<256, 4>(g, ta, tb, grid, splits, stream);
    case 192: return dispatch_major<192, 5>(g, ta, tb, grid, splits, stream);
    case 128: return dispatch_major<128, 6>(g, ta, tb, grid, splits, stream);
    default: return dispatch_major<64, 8>(g, ta, tb, grid, splits, stream);
  }
}
