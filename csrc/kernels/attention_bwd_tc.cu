// Flash attention backward on the 5th-generation tensor cores: two kernels from one template, no atomics.
//
//   MODE_DKV  one CTA owns 128 keys of one (batch, kv head) and walks over the query tiles that see them
//             (all query heads of the group):  dV += P^T dO,  dK += dS^T Q   (accumulators stay in TMEM for the whole walk)
//   MODE_DQ   one CTA owns 128 queries of one (batch, head) and walks over the key tiles they see:  dQ += dS K
//
// Per (query tile, key tile) pair, in both modes:
//   S  = Q K^T, dP = dO V^T        tcgen05.mma (SS) into two 128-column TMEM accumulators
//   P  = exp2(S * scale * log2e - lse * log2e), dS = P * (dP - delta)
//                                   sixteen warps; a thread owns one query row (its TMEM lane) and 32 of the 128 keys;
//                                   P and dS go to shared memory as bf16 in the 128-byte-swizzled layout
//   dV / dK / dQ                    tcgen05.mma (SS) reading P and dS either K-major (dQ) or transposed through an
//                                   MN-major descriptor (dV, dK), and dO / Q / K MN-major straight from their row layout
// The tiles of the walk arrive by TMA (4-D maps over the strided [batch, seq, head, dim] views), double buffered when
// shared memory allows.  The S / dP products of step t+1 are issued before the dV / dK / dQ products of step t, so the
// tensor cores work on them while the warps are still in step t's exponentials.
//
// Roles: warps 0-15 softmax / dS / epilogue (four lane quarters x four 32-key column groups), warp 16 TMA producer,
// warp 17 MMA issuer.  Every wait is bounded.
// Same semantics as the mma.sync backward in attention.cu (causal alignment to the end of the keys, GQA).
#include "attention.h"

#include "rb_common.cuh"

namespace rb {

constexpr int kBtTile = 128;
constexpr int kBtColGroups = 2;                    // compute warps = 4 lane quarters x this many column groups
constexpr int kBtComputeWarps = 4 * kBtColGroups;
constexpr int kBtThreads = 32 * (kBtComputeWarps + 2);
constexpr int kBtColsPerGroup = kBtTile / kBtColGroups;   // keys per compute thread and step
constexpr float kBtLog2e = 1.4426950408889634f;
constexpr int MODE_DKV = 0;
constexpr int MODE_DQ = 1;

struct BtParams {
  const float* lse;
  const float* delta;
  __nv_bfloat16* out0;      // MODE_DKV: dK;  MODE_DQ: dQ
  __nv_bfloat16* out1;      // MODE_DKV: dV
  long long o0_bs, o0_rs, o0_hs, o1_bs, o1_rs, o1_hs;
  int seq_q, seq_k, heads, kv_heads, causal, batch;
  float scale;
};

__device__ __forceinline__ float bt_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D, int MODE>
struct BtSmem {
  static constexpr int kHalf = kBtTile * 128;                  // 128 rows x 128 B: one 64-column swizzle atom column
  static constexpr int kTileBytes = (D / 64) * kHalf;          // one [128, D] operand tile
  // streamed pair double buffered when it fits: always for head dim 64, for head dim 128 only in MODE_DQ (no P buffer)
  static constexpr int kStages = (D == 64 || MODE == MODE_DQ) ? 2 : 1;
  // the owned ("resident") pair of the NEXT work item is prefetched while the current one is processed when it fits
  static constexpr int kResStages = (D == 64) ? 2 : 1;
  static constexpr int kRes0 = 0;                              // resident pair: (K, V) in MODE_DKV, (Q, dO) in MODE_DQ
  static constexpr int kRes1 = kRes0 + kTileBytes;             // (per resident stage: two tiles)
  static constexpr int kStream = kResStages * 2 * kTileBytes;  // per stage: two tiles
  static constexpr int kDs = kStream + kStages * 2 * kTileBytes;
  static constexpr int kP = kDs + 2 * kHalf;
  static constexpr int kBar = kP + (MODE == MODE_DKV ? 2 * kHalf : 0);
  static constexpr int kNumBars = 16;
  static constexpr int kTotal = kBar + kNumBars * 8 + 16;
};

template <int D>
__global__ void __launch_bounds__(256)
attn_delta_tc_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                     long long bs, long long rs, long long hs, int heads, int seq_q) {
  // delta[b, h, r] = sum_d dO * O.  D / 8 adjacent lanes share a row (one 16-byte load of each tensor per lane).
  constexpr int TPR = D / 8;                       // threads per row: 8 or 16
  constexpr int RPB = 256 / TPR;                   // rows per block
  const int b = blockIdx.y;
  const long long idx = static_cast<long long>(blockIdx.x) * RPB + threadIdx.x / TPR;
  const int part = threadIdx.x % TPR;
  float acc = 0.f;
  const bool live = idx < static_cast<long long>(heads) * seq_q;
  int h = 0, r = 0;
  if (live) {
    // rows are walked (row, head)-major so that neighbouring threads read neighbouring memory in a [B, S, H, D] tensor
    r = static_cast<int>(idx / heads);
    h = static_cast<int>(idx % heads);
    const long long off = b * bs + h * hs + static_cast<long long>(r) * rs + part * 8;
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(o + off));
    const uint4 g = __ldg(reinterpret_cast<const uint4*>(d_o + off));
    const uint32_t* ua = reinterpret_cast<const uint32_t*>(&a);
    const uint32_t* ug = reinterpret_cast<const uint32_t*>(&g);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = unpack_bf16x2(ua[j]), y = unpack_bf16x2(ug[j]);
      acc = fmaf(x.x, y.x, acc);
      acc = fmaf(x.y, y.y, acc);
    }
  }
#pragma unroll
  for (int m = TPR / 2; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
  if (live && part == 0) delta[(static_cast<long long>(b) * heads + h) * seq_q + r] = acc;
}

template <int D, int MODE>
__global__ void __launch_bounds__(kBtThreads, 1)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, BtParams p,
                   unsigned int* status) {
  using L = BtSmem<D, MODE>;
  constexpr int STAGES = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  const uint32_t b0 = smem_u32(bars);
  const uint32_t bar_tfull = b0 + 8, bar_tempty = b0 + 24, bar_sdp_full = b0 + 40, bar_sdp_empty = b0 + 48,
                 bar_p_full = b0 + 56, bar_p_empty = b0 + 64, bar_acc_full = b0 + 72, bar_res = b0 + 104;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const uint32_t bar_res_empty = b0 + 80, bar_acc_empty = b0 + 96;      // bar_res / bar_res_empty: two slots each
  constexpr int RS = L::kResStages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.heads / p.kv_heads;
  const int shift = p.seq_k - p.seq_q;
  const int n_q_tiles = (p.seq_q + kBtTile - 1) / kBtTile;
  const int n_k_tiles = (p.seq_k + kBtTile - 1) / kBtTile;

  // Work items: one owned tile of one (head, batch).  A CTA is persistent and takes items blockIdx.x, + gridDim.x, ...;
  // items are numbered so that the long walks come first (MODE_DKV: early key tiles, MODE_DQ: late query tiles).
  struct Work { int own0, walk_first, walk_count, n_it, head_q0, head_k, b; };
  const int n_own = MODE == MODE_DKV ? n_k_tiles : n_q_tiles;
  const int ny = MODE == MODE_DKV ? p.kv_heads : p.heads;
  const int total_items = n_own * ny * p.batch;
  auto get_work = [&](int item, Work& w) {
    const int per_tile = ny * p.batch;
    const int tw = item / per_tile;
    const int yz = item - tw * per_tile;
    const int y = yz % ny;
    w.b = yz / ny;
    const int blk = (MODE == MODE_DKV || !p.causal) ? tw : n_own - 1 - tw;
    w.own0 = blk * kBtTile;
    w.walk_first = 0;
    if (MODE == MODE_DKV) {
      w.head_k = y;
      w.head_q0 = y * group;
      if (p.causal && w.own0 - shift > 0) w.walk_first = (w.own0 - shift) / kBtTile;
      w.walk_count = n_q_tiles - w.walk_first;
      if (w.walk_count < 0) w.walk_count = 0;
      w.n_it = w.walk_count * group;
    } else {
      w.head_q0 = y;
      w.head_k = y / group;
      w.walk_count = n_k_tiles;
      if (p.causal) {
        const int lim = (w.own0 + kBtTile - 1 + shift) / kBtTile + 1;
        if (lim < w.walk_count) w.walk_count = lim;
      }
      w.n_it = w.walk_count;
    }
  };
  auto walk_decode = [&](const Work& w, int it, int& hq, int& q0, int& k0) {
    if (MODE == MODE_DKV) {
      const int g = it / w.walk_count;
      hq = w.head_q0 + g;
      q0 = (w.walk_first + it - g * w.walk_count) * kBtTile;
      k0 = w.own0;
    } else {
      hq = w.head_q0;
      q0 = w.own0;
      k0 = it * kBtTile;
    }
  };

  constexpr uint32_t kTmemCols = 512;           // S [0,128)  dP [128,256)  accumulators from 256
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_res + 8 * s, 1);
      mbar_init(bar_res_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, 1);
    }
    mbar_init(bar_sdp_full, 1);
    mbar_init(bar_sdp_empty, kBtComputeWarps);
    mbar_init(bar_p_full, kBtComputeWarps);
    mbar_init(bar_p_empty, 1);
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, kBtComputeWarps);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == kBtComputeWarps + 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + 128, tmem_acc0 = tmem_base + 256, tmem_acc1 = tmem_base + 256 + D;

  const uint32_t sRes0 = sbase + L::kRes0, sRes1 = sbase + L::kRes1, sStream = sbase + L::kStream;
  const uint32_t sDs = sbase + L::kDs, sP = sbase + L::kP;

  // Running counters: `wi` counts this CTA's work items, `git` its steps over all items, `ai` its items that have at
  // least one step; the barrier phases follow them, so every role derives the same parities independently.
  if (warp == kBtComputeWarps) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      uint32_t git = 0, wi = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++wi) {
        Work w;
        get_work(item, w);
        // the resident pair is free once the previous item's products have all been issued and completed
        const uint32_t rsl = wi % RS;
        if (!mbar_wait(bar_res_empty + 8 * rsl, ((wi / RS) & 1) ^ 1, abort_flag, status, 40)) break;
        const uint32_t rfull = bar_res + 8 * rsl;
        const uint32_t r0 = sRes0 + rsl * 2 * L::kTileBytes, r1 = sRes1 + rsl * 2 * L::kTileBytes;
        mbar_arrive_expect_tx(rfull, 2 * L::kTileBytes);
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf) {
          if (MODE == MODE_DKV) {
            tma_load_4d(r0 + hf * L::kHalf, &tmK, hf * 64, w.head_k, w.own0, w.b, rfull);
            tma_load_4d(r1 + hf * L::kHalf, &tmV, hf * 64, w.head_k, w.own0, w.b, rfull);
          } else {
            tma_load_4d(r0 + hf * L::kHalf, &tmQ, hf * 64, w.head_q0, w.own0, w.b, rfull);
            tma_load_4d(r1 + hf * L::kHalf, &tmdO, hf * 64, w.head_q0, w.own0, w.b, rfull);
          }
        }
        for (int it = 0; it < w.n_it; ++it, ++git) {
          const uint32_t s = git % STAGES;
          if (!mbar_wait(bar_tempty + 8 * s, ((git / STAGES) & 1) ^ 1, abort_flag, status, 41)) { ok = false; break; }
          int hq, q0, k0;
          walk_decode(w, it, hq, q0, k0);
          mbar_arrive_expect_tx(bar_tfull + 8 * s, 2 * L::kTileBytes);
          const uint32_t d0 = sStream + s * 2 * L::kTileBytes, d1 = d0 + L::kTileBytes;
#pragma unroll
          for (int hf = 0; hf < D / 64; ++hf) {
            if (MODE == MODE_DKV) {
              tma_load_4d(d0 + hf * L::kHalf, &tmQ, hf * 64, hq, q0, w.b, bar_tfull + 8 * s);
              tma_load_4d(d1 + hf * L::kHalf, &tmdO, hf * 64, hq, q0, w.b, bar_tfull + 8 * s);
            } else {
              tma_load_4d(d0 + hf * L::kHalf, &tmK, hf * 64, w.head_k, k0, w.b, bar_tfull + 8 * s);
              tma_load_4d(d1 + hf * L::kHalf, &tmV, hf * 64, w.head_k, k0, w.b, bar_tfull + 8 * s);
            }
          }
        }
      }
    }
  } else if (warp == kBtComputeWarps + 1) {
    if (lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_t = umma_idesc_bf16(128, D, 1, 1);      // dV, dK: A (P / dS) and B (dO / Q) both MN-major
      constexpr uint32_t idesc_q = umma_idesc_bf16(128, D, 0, 1);      // dQ: A = dS K-major, B = K MN-major
      uint32_t res_off = 0;                            // byte offset of the current item's resident pair
      auto issue_sdp = [&](uint32_t g) -> bool {      // g: running step index
        const uint32_t s = g % STAGES;
        if (!mbar_wait(bar_tfull + 8 * s, (g / STAGES) & 1, abort_flag, status, 42)) return false;
        if (!mbar_wait(bar_sdp_empty, (g & 1) ^ 1, abort_flag, status, 43)) return false;
        tc_fence_after();
        const uint32_t t0 = sStream + s * 2 * L::kTileBytes, t1 = t0 + L::kTileBytes;
        const uint32_t aQ = MODE == MODE_DKV ? t0 : sRes0 + res_off, adO = MODE == MODE_DKV ? t1 : sRes1 + res_off;
        const uint32_t bK = MODE == MODE_DKV ? sRes0 + res_off : t0, bV = MODE == MODE_DKV ? sRes1 + res_off : t1;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * L::kHalf + (ks & 3) * 32;
          umma_bf16_ss(tmem_s, umma_smem_desc_sw128(aQ + off, 16, 1024), umma_smem_desc_sw128(bK + off, 16, 1024), idesc_s,
                       ks != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * L::kHalf + (ks & 3) * 32;
          umma_bf16_ss(tmem_dp, umma_smem_desc_sw128(adO + off, 16, 1024), umma_smem_desc_sw128(bV + off, 16, 1024), idesc_s,
                       ks != 0 ? 1u : 0u);
        }
        umma_commit(bar_sdp_full);
        return true;
      };
      uint32_t git = 0, wi = 0, ai = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++wi) {
        Work w;
        get_work(item, w);
        const uint32_t rsl = wi % RS;
        res_off = rsl * 2 * L::kTileBytes;
        if (!mbar_wait(bar_res + 8 * rsl, (wi / RS) & 1, abort_flag, status, 44)) break;
        if (w.n_it > 0) {
          // the warps have read out the previous item's accumulators
          if (!mbar_wait(bar_acc_empty, (ai & 1) ^ 1, abort_flag, status, 49)) break;
          ok = issue_sdp(git);
        }
        for (int it = 0; it < w.n_it && ok; ++it, ++git) {
          const uint32_t s = git % STAGES;
          // With two stages the next S / dP pair goes to the tensor cores ahead of this step's accumulations; with one
          // stage its operands can only be loaded after those accumulations have released the buffer.
          if (STAGES == 2 && it + 1 < w.n_it) {
            ok = issue_sdp(git + 1);
            if (!ok) break;
          }
          if (!mbar_wait(bar_p_full, git & 1, abort_flag, status, 45)) { ok = false; break; }
          tc_fence_after();
          const uint32_t t0 = sStream + s * 2 * L::kTileBytes, t1 = t0 + L::kTileBytes;
          if (MODE == MODE_DKV) {
#pragma unroll
            for (int ks = 0; ks < kBtTile / 16; ++ks) {      // dK += dS^T Q   (k = query rows)
              umma_bf16_ss(tmem_acc0, umma_smem_desc_sw128(sDs + ks * 2048, L::kHalf, 1024),
                           umma_smem_desc_sw128(t0 + ks * 2048, L::kHalf, 1024), idesc_t, (it != 0 || ks != 0) ? 1u : 0u);
            }
#pragma unroll
            for (int ks = 0; ks < kBtTile / 16; ++ks) {      // dV += P^T dO
              umma_bf16_ss(tmem_acc1, umma_smem_desc_sw128(sP + ks * 2048, L::kHalf, 1024),
                           umma_smem_desc_sw128(t1 + ks * 2048, L::kHalf, 1024), idesc_t, (it != 0 || ks != 0) ? 1u : 0u);
            }
          } else {
#pragma unroll
            for (int ks = 0; ks < kBtTile / 16; ++ks) {      // dQ += dS K     (k = keys)
              umma_bf16_ss(tmem_acc0, umma_smem_desc_sw128(sDs + (ks >> 2) * L::kHalf + (ks & 3) * 32, 16, 1024),
                           umma_smem_desc_sw128(t0 + ks * 2048, L::kHalf, 1024), idesc_q, (it != 0 || ks != 0) ? 1u : 0u);
            }
          }
          umma_commit(bar_p_empty);
          umma_commit(bar_tempty + 8 * s);
          if (STAGES == 1 && it + 1 < w.n_it) ok = issue_sdp(git + 1);
        }
        if (!ok) break;
        if (w.n_it > 0) {
          umma_commit(bar_acc_full);
          ++ai;
        }
        umma_commit(bar_res_empty + 8 * rsl);     // every product that reads this resident pair has completed by then
      }
    }
  } else {
    // ------------------------------------------------------------------ P / dS and the read-out of every item
    const int qtr = warp & 3, cg = warp >> 2;              // TMEM lane quarter, column group
    constexpr int GC = kBtColsPerGroup;                    // columns (keys) per thread and step: 64 or 32
    const int row = qtr * 32 + lane;                       // query row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    const float sl2 = p.scale * kBtLog2e;
    bool ok = true;
    uint32_t git = 0, ai = 0;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      Work w;
      get_work(item, w);
      const int b = w.b;
      // log-sum-exp and delta of this thread's row are fetched one step ahead: the load latency hides behind a step
      auto load_stats = [&](int it, float& lse2, float& dlt) {
        int hq, q0, k0;
        walk_decode(w, it, hq, q0, k0);
        const int q_idx = q0 + row;
        if (q_idx < p.seq_q) {
          const long long stat = (static_cast<long long>(b) * p.heads + hq) * p.seq_q + q_idx;
          lse2 = __ldg(p.lse + stat) * kBtLog2e;
          dlt = __ldg(p.delta + stat);
        } else {
          lse2 = 0.f;
          dlt = 0.f;
        }
      };
      float lse2_next = 0.f, dlt_next = 0.f;
      if (w.n_it > 0) load_stats(0, lse2_next, dlt_next);
      for (int it = 0; it < w.n_it && ok; ++it, ++git) {
        int hq, q0, k0;
        walk_decode(w, it, hq, q0, k0);
        const int q_idx = q0 + row;
        const bool q_ok = q_idx < p.seq_q;
        const float lse2 = lse2_next, dlt = dlt_next;
        if (it + 1 < w.n_it) load_stats(it + 1, lse2_next, dlt_next);
        const int key_lim = q_ok ? (p.causal ? min(p.seq_k - 1, q_idx + shift) : p.seq_k - 1) : -1;   // last visible key
        const int kbase = k0 + cg * GC;
        const bool need_mask = (kbase + GC - 1 > key_lim);
        if (!mbar_wait(bar_sdp_full, git & 1, abort_flag, status, 46)) { ok = false; break; }
        tc_fence_after();
        uint32_t pp[GC / 2], ds[GC / 2];                     // GC columns each, packed bf16 pairs
        // 16 columns of S and of dP per step; the loads of step c + 1 are in flight while step c is computed
        const uint32_t ts = tmem_s + lane_off + cg * GC, td = tmem_dp + lane_off + cg * GC;
        uint32_t rs[2][16], rd[2][16];
        tmem_ld_32x16(ts, rs[0]);
        tmem_ld_32x16(td, rd[0]);
#pragma unroll
        for (int c = 0; c < GC / 16; ++c) {
          tmem_ld_wait();
          if (c + 1 < GC / 16) {
            tmem_ld_32x16(ts + (c + 1) * 16, rs[(c + 1) & 1]);
            tmem_ld_32x16(td + (c + 1) * 16, rd[(c + 1) & 1]);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float p0 = bt_ex2(fmaf(__uint_as_float(rs[c & 1][2 * i]), sl2, -lse2));
            float p1 = bt_ex2(fmaf(__uint_as_float(rs[c & 1][2 * i + 1]), sl2, -lse2));
            if (need_mask) {
              const int key = kbase + c * 16 + 2 * i;
              if (key > key_lim) p0 = 0.f;
              if (key + 1 > key_lim) p1 = 0.f;
            }
            const float d0 = p0 * (__uint_as_float(rd[c & 1][2 * i]) - dlt);
            const float d1 = p1 * (__uint_as_float(rd[c & 1][2 * i + 1]) - dlt);
            pp[c * 8 + i] = pack_bf16x2(p0, p1);
            ds[c * 8 + i] = pack_bf16x2(d0, d1);
          }
        }
        // S and dP are in registers: the next pair of products may overwrite them
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sdp_empty);
        // the previous step's dV / dK / dQ products have finished reading P and dS
        if (!mbar_wait(bar_p_empty, (git & 1) ^ 1, abort_flag, status, 47)) { ok = false; break; }
        // 64 keys are one 128-byte-swizzled atom (row `row`, eight 16-byte chunks); this thread owns GC / 8 of the chunks
        constexpr int CH = GC / 8;
        const int atom = (cg * GC) / 64, ch0 = ((cg * GC) % 64) / 8;
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
          const uint32_t off = atom * L::kHalf + row * 128 + (((ch0 + ch) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sDs + off), "r"(ds[4 * ch]), "r"(ds[4 * ch + 1]),
                       "r"(ds[4 * ch + 2]), "r"(ds[4 * ch + 3])
                       : "memory");
          if (MODE == MODE_DKV) {
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sP + off), "r"(pp[4 * ch]), "r"(pp[4 * ch + 1]),
                         "r"(pp[4 * ch + 2]), "r"(pp[4 * ch + 3])
                         : "memory");
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_full);
      }
      if (!ok) break;

      // ---- read-out: TMEM lane = key (MODE_DKV) or query (MODE_DQ) row of the owned tile; this group's share of D
      const bool have = w.n_it > 0;
      if (have && !mbar_wait(bar_acc_full, ai & 1, abort_flag, status, 48)) { ok = false; break; }
      tc_fence_after();
      const int r_idx = w.own0 + row;
      const int limit = MODE == MODE_DKV ? p.seq_k : p.seq_q;
      const int head_out = MODE == MODE_DKV ? w.head_k : w.head_q0;
      constexpr int CW = D / kBtColGroups;                 // output columns per column group (16, 32 or 64)
#pragma unroll
      for (int which = 0; which < (MODE == MODE_DKV ? 2 : 1); ++which) {
        const uint32_t tacc = which == 0 ? tmem_acc0 : tmem_acc1;
        const float mul = which == 0 ? p.scale : 1.f;      // dK and dQ carry the softmax scale, dV does not
        __nv_bfloat16* base = which == 0 ? p.out0 : p.out1;
        const long long bs = which == 0 ? p.o0_bs : p.o1_bs, rs_ = which == 0 ? p.o0_rs : p.o1_rs,
                        hs = which == 0 ? p.o0_hs : p.o1_hs;
#pragma unroll
        for (int c = 0; c < CW / 16; ++c) {
          uint32_t r[16];
          if (have) {
            tmem_ld_32x16(tacc + lane_off + cg * CW + c * 16, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = 0u;
          }
          if (r_idx < limit) {
            __nv_bfloat16* op = base + b * bs + head_out * hs + static_cast<long long>(r_idx) * rs_ + cg * CW + c * 16;
#pragma unroll
            for (int v4 = 0; v4 < 2; ++v4) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[v4 * 8 + 0]) * mul, __uint_as_float(r[v4 * 8 + 1]) * mul);
              o.y = pack_bf16x2(__uint_as_float(r[v4 * 8 + 2]) * mul, __uint_as_float(r[v4 * 8 + 3]) * mul);
              o.z = pack_bf16x2(__uint_as_float(r[v4 * 8 + 4]) * mul, __uint_as_float(r[v4 * 8 + 5]) * mul);
              o.w = pack_bf16x2(__uint_as_float(r[v4 * 8 + 6]) * mul, __uint_as_float(r[v4 * 8 + 7]) * mul);
              reinterpret_cast<uint4*>(op)[v4] = o;
            }
          }
        }
      }
      if (have) {
        // the accumulators are in registers / memory: the next item's products may overwrite them
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty);
        ++ai;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kBtComputeWarps + 1) {
    if (*abort_flag) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace rb

namespace {
const CUtensorMap* bt_map(const void* base, const long long* strides, int seq, int heads, int batch, int D, int* err) {
  long long s[3] = {strides[0] > 0 ? strides[0] : 8, strides[1] > 0 ? strides[1] : D, strides[2] > 0 ? strides[2] : D};
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)heads, (uint64_t)seq, (uint64_t)batch};
  const uint64_t str[3] = {(uint64_t)s[2] * 2, (uint64_t)s[1] * 2, (uint64_t)s[0] * 2};
  const uint32_t box[4] = {64, 1, (uint32_t)rb::kBtTile, 1};
  return rbhost::get_tmap_4d(base, 2, dims, str, box, 1, err);
}

template <int D, int MODE>
int bt_launch(const CUtensorMap* tq, const CUtensorMap* tk, const CUtensorMap* tv, const CUtensorMap* tdo,
              const rb::BtParams& p, dim3 grid, cudaStream_t stream) {
  auto kern = rb::attn_bwd_tc_kernel<D, MODE>;
  const int smem = rb::BtSmem<D, MODE>::kTotal + 1024;
  static bool cfg_dev[64] = {false};
    bool& cfg = cfg_dev[rbhost::device_slot()];
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    cfg = true;
  }
  kern<<<grid, rb::kBtThreads, smem, stream>>>(*tq, *tk, *tv, *tdo, p, rbhost::status_ptr());
  return static_cast<int>(cudaGetLastError());
}
}  // namespace

// delta[b, h, r] = sum_d dO * O (fp32), the row term of the softmax gradient; shared by both tcgen05 backward paths.
RB_API int rb_attention_delta_tc(const RbAttnArgs* a, void* stream_v) {
  const int D = a->head_dim;
  if (D != 64 && D != 128) return -9;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const long long rows = static_cast<long long>(a->heads) * a->seq_q;
  const int rows_per_block = 256 / (D / 8);
  dim3 dgrid(static_cast<unsigned>((rows + rows_per_block - 1) / rows_per_block), a->batch);
  const __nv_bfloat16* o = reinterpret_cast<const __nv_bfloat16*>(a->o);
  const __nv_bfloat16* d_o = reinterpret_cast<const __nv_bfloat16*>(a->d_o);
  if (D == 64)
    rb::attn_delta_tc_kernel<64><<<dgrid, 256, 0, stream>>>(o, d_o, a->delta, a->o_strides[0], a->o_strides[1],
                                                             a->o_strides[2], a->heads, a->seq_q);
  else
    rb::attn_delta_tc_kernel<128><<<dgrid, 256, 0, stream>>>(o, d_o, a->delta, a->o_strides[0], a->o_strides[1],
                                                              a->o_strides[2], a->heads, a->seq_q);
  return static_cast<int>(cudaGetLastError());
}

// Backward pass on the tcgen05 path (three launches: delta, dK/dV, dQ).  Returns -9 when the problem is outside what
// these kernels take (the caller then uses rb_attention_bwd).
RB_API int rb_attention_bwd_tc(const RbAttnArgs* a, void* stream_v) {
  if (a->kv_lens) return -9;                 // key-padding lengths: only the second-generation kernels take them
  if (a->batch <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads) return -1;
  if (a->head_dim != 64 && a->head_dim != 128) return -9;
  if (a->seq_q <= 0 || a->seq_k <= 0 || (a->causal && a->seq_q > a->seq_k)) return -1;
  if (!a->lse || !a->delta) return -2;
  const void* ptrs[8] = {a->q, a->k, a->v, a->o, a->d_o, a->dq, a->dk, a->dv};
  for (int i = 0; i < 8; ++i)
    if (!ptrs[i] || (reinterpret_cast<uintptr_t>(ptrs[i]) & 15)) return -9;
  const long long* strs[7] = {a->q_strides, a->k_strides, a->v_strides, a->o_strides, a->dq_strides, a->dk_strides, a->dv_strides};
  for (int i = 0; i < 7; ++i)
    for (int j = 0; j < 3; ++j)
      if (strs[i][j] % 8) return -9;
  const int D = a->head_dim;
  int err = 0;
  const CUtensorMap* tq = bt_map(a->q, a->q_strides, a->seq_q, a->heads, a->batch, D, &err);
  const CUtensorMap* tk = bt_map(a->k, a->k_strides, a->seq_k, a->kv_heads, a->batch, D, &err);
  const CUtensorMap* tv = bt_map(a->v, a->v_strides, a->seq_k, a->kv_heads, a->batch, D, &err);
  const CUtensorMap* tdo = bt_map(a->d_o, a->o_strides, a->seq_q, a->heads, a->batch, D, &err);
  if (!tq || !tk || !tv || !tdo) return err ? err : -5;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);

  rb_attention_delta_tc(a, stream_v);

  rb::BtParams p;
  p.lse = a->lse; p.delta = a->delta;
  p.seq_q = a->seq_q; p.seq_k = a->seq_k; p.heads = a->heads; p.kv_heads = a->kv_heads; p.causal = a->causal;
  p.batch = a->batch;
  p.scale = a->scale;
  // dK / dV
  p.out0 = reinterpret_cast<__nv_bfloat16*>(a->dk); p.out1 = reinterpret_cast<__nv_bfloat16*>(a->dv);
  p.o0_bs = a->dk_strides[0]; p.o0_rs = a->dk_strides[1]; p.o0_hs = a->dk_strides[2];
  p.o1_bs = a->dv_strides[0]; p.o1_rs = a->dv_strides[1]; p.o1_hs = a->dv_strides[2];
  // persistent CTAs: one per SM, each walks over work items (owned tile, head, batch)
  const int sms = rbhost::device_sm_count();
  const long long kv_items = static_cast<long long>((a->seq_k + rb::kBtTile - 1) / rb::kBtTile) * a->kv_heads * a->batch;
  dim3 kvgrid(static_cast<unsigned>(kv_items < sms ? kv_items : sms));
  int rc = D == 64 ? bt_launch<64, rb::MODE_DKV>(tq, tk, tv, tdo, p, kvgrid, stream)
                   : bt_launch<128, rb::MODE_DKV>(tq, tk, tv, tdo, p, kvgrid, stream);
  if (rc != 0) return rc;
  // dQ
  p.out0 = reinterpret_cast<__nv_bfloat16*>(a->dq); p.out1 = nullptr;
  p.o0_bs = a->dq_strides[0]; p.o0_rs = a->dq_strides[1]; p.o0_hs = a->dq_strides[2];
  const long long q_items = static_cast<long long>((a->seq_q + rb::kBtTile - 1) / rb::kBtTile) * a->heads * a->batch;
  dim3 qgrid(static_cast<unsigned>(q_items < sms ? q_items : sms));
  return D == 64 ? bt_launch<64, rb::MODE_DQ>(tq, tk, tv, tdo, p, qgrid, stream)
                 : bt_launch<128, rb::MODE_DQ>(tq, tk, tv, tdo, p, qgrid, stream);
}
