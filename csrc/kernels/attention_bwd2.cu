// Flash attention backward on the 5th-generation tensor cores, second version: P and dS never touch shared memory.
//
// Two kernels from one template, no atomics, bit-reproducible:
//
//   MODE_DQ   a CTA owns 128 queries of one (batch, head) (Q, dO resident in shared memory) and walks over the key
//             tiles they see.  Per step
//                 S  = Q K^T,  dP = dO V^T          tcgen05.mma (SS), accumulators in TMEM (dP double buffered)
//                 dS = exp2(S c - lse) (dP - delta) eight warps, query row = TMEM lane; dS goes back to TMEM as packed
//                                                   bf16 over the dP buffer
//                 dQ += dS K                        tcgen05.mma, A operand dS read from TMEM (TS form), K MN-major
//   MODE_DKV  a CTA owns 128 keys of one (batch, kv head) (K, V resident) and walks over the query tiles that see them
//             (all query heads of the group).  The products are formed TRANSPOSED, so that the key is the TMEM lane:
//                 S^T = K Q^T,  dP^T = V dO^T
//                 P^T -> TMEM over S^T,  dV += P^T dO      (TS form, dO MN-major)
//                 dS^T -> TMEM over dP^T, dK += dS^T Q     (TS form, Q MN-major)
//             The log-sum-exp and delta of the step's 128 queries vary along a thread's row here; they are staged in
//             shared memory one step ahead and read as broadcasts.  With head dim 64 S^T is double buffered.
//
// Because every product that overwrites a TMEM buffer is issued by the one MMA thread after the product that last read
// it, and tcgen05.mma instructions of one thread execute in issue order, no "buffer free" handshake is needed for the
// aliased P / dS operands; the only waits are "operand tile landed", "scores ready", "probabilities written".
// Roles: warps 0-7 compute (lane quarter = warp & 3, column half = warp >> 2), warp 8 TMA producer, warp 9 MMA issuer.
// CTAs are persistent and walk over work items; every wait is bounded.
//
// Same semantics as the other backward kernels (causal alignment to the end of the keys, GQA); replaces the
// reference's dense attention gradient (crates/autodiff/src/lib.rs:645-806 applied to crates/nn/src/attention.rs:640-836).
#include "attention.h"

#include "rb_common.cuh"

namespace rb {

constexpr int kB2Tile = 128;
constexpr int kB2ComputeWarps = 8;
constexpr int kB2Threads = 32 * (kB2ComputeWarps + 2);
constexpr float kB2Log2e = 1.4426950408889634f;
constexpr int B2_DKV = 0;
constexpr int B2_DQ = 1;

struct B2Params {
  const float* lse;
  const float* delta;
  __nv_bfloat16* out0;      // B2_DKV: dK;  B2_DQ: dQ
  __nv_bfloat16* out1;      // B2_DKV: dV
  long long o0_bs, o0_rs, o0_hs, o1_bs, o1_rs, o1_hs;
  int seq_q, seq_k, heads, kv_heads, causal, batch;
  float scale;
  const int* kv_lens;       // optional [batch]: number of real keys (the rest of seq_k is padding)
};

__device__ __forceinline__ float b2_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void b2_bar_compute() {            // the 256 compute threads only
  asm volatile("bar.sync 1, 256;" ::: "memory");
}

template <int D, int MODE>
struct B2Smem {
  static constexpr int kHalf = kB2Tile * 128;                  // 128 rows x 128 B: one 64-column swizzle atom
  static constexpr int kTileBytes = (D / 64) * kHalf;          // one [128, D] operand tile
  static constexpr int kResStages = D == 64 ? 2 : 1;           // owned pair of the next work item prefetched
  static constexpr int kStages = D == 64 ? 3 : 2;              // streamed pairs in flight
  static constexpr int kRes = 0;
  static constexpr int kStream = kResStages * 2 * kTileBytes;
  static constexpr int kStats = kStream + kStages * 2 * kTileBytes;     // [2 steps][lse2 | delta][128] fp32
  static constexpr int kBar = kStats + 2 * 2 * 128 * 4;
  // + s_full[2], s_empty, dp_full[2], p_full[2], ds_full[2], acc_full, acc_empty
  static constexpr int kNumBars = 2 * kResStages + 2 * kStages + 11;
  static constexpr int kTotal = kBar + kNumBars * 8 + 16;
  // TMEM columns
  static constexpr int kSBufs = (MODE == B2_DKV && D == 64) ? 2 : 1;    // S (S^T) buffers
  static constexpr int kDpBufs = MODE == B2_DQ ? 2 : 1;                 // dP buffers
  static constexpr int kColS = 0;
  static constexpr int kColDp = kColS + 128 * kSBufs;
  static constexpr int kColAcc0 = kColDp + 128 * kDpBufs;
  static constexpr int kColAcc1 = kColAcc0 + D;
  static_assert(kColAcc0 + (MODE == B2_DKV ? 2 : 1) * D <= 512, "TMEM budget");
};

template <int D, int MODE>
__global__ void __launch_bounds__(kB2Threads, 1)
attn_bwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, B2Params p,
                 unsigned int* status) {
  using L = B2Smem<D, MODE>;
  constexpr int ST = L::kStages, RS = L::kResStages, SB = L::kSBufs, DB = L::kDpBufs;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  const uint32_t b0 = smem_u32(bars);
  const uint32_t bar_res = b0, bar_res_empty = bar_res + 8 * RS, bar_tfull = bar_res_empty + 8 * RS,
                 bar_tempty = bar_tfull + 8 * ST, bar_sfull = bar_tempty + 8 * ST /* [2] */, bar_sempty = bar_sfull + 16,
                 bar_dpfull = bar_sempty + 8 /* [2] */, bar_pfull = bar_dpfull + 16 /* [2] */, bar_dsfull = bar_pfull + 16 /* [2] */,
                 bar_accfull = bar_dsfull + 16, bar_accempty = bar_accfull + 8;
  static_assert(2 * RS + 2 * ST + 11 == L::kNumBars, "barrier count");
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  float* stats = reinterpret_cast<float*>(smem + L::kStats);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.heads / p.kv_heads;
  const int shift = p.seq_k - p.seq_q;
  const int n_q_tiles = (p.seq_q + kB2Tile - 1) / kB2Tile;
  const int n_k_tiles = (p.seq_k + kB2Tile - 1) / kB2Tile;

  // Work items: one owned tile of one (head, batch); a CTA takes items blockIdx.x, + gridDim.x, ...  Long walks first.
  struct Work { int own0, walk_first, walk_count, n_it, head_q0, head_k, b, kv_len; };
  const int n_own = MODE == B2_DKV ? n_k_tiles : n_q_tiles;
  const int ny = MODE == B2_DKV ? p.kv_heads : p.heads;
  const int total_items = n_own * ny * p.batch;
  auto get_work = [&](int item, Work& w) {
    const int per_tile = ny * p.batch;
    const int tw = item / per_tile;
    const int yz = item - tw * per_tile;
    const int y = yz % ny;
    w.b = yz / ny;
    const int blk = (MODE == B2_DKV || !p.causal) ? tw : n_own - 1 - tw;
    w.own0 = blk * kB2Tile;
    w.walk_first = 0;
    // padded keys (positions >= kv_len) are invisible: their dK / dV are zero and no query walks over them
    w.kv_len = p.kv_lens ? max(0, min(p.seq_k, p.kv_lens[w.b])) : p.seq_k;
    if (MODE == B2_DKV) {
      w.head_k = y;
      w.head_q0 = y * group;
      if (p.causal && w.own0 - shift > 0) w.walk_first = (w.own0 - shift) / kB2Tile;
      w.walk_count = n_q_tiles - w.walk_first;
      if (w.walk_count < 0 || w.own0 >= w.kv_len) w.walk_count = 0;
      w.n_it = w.walk_count * group;
    } else {
      w.head_q0 = y;
      w.head_k = y / group;
      w.walk_count = (w.kv_len + kB2Tile - 1) / kB2Tile;
      if (p.causal) {
        const int lim = (w.own0 + kB2Tile - 1 + shift) / kB2Tile + 1;
        if (lim < w.walk_count) w.walk_count = lim;
      }
      w.n_it = w.walk_count;
    }
  };
  auto walk_decode = [&](const Work& w, int it, int& hq, int& q0, int& k0) {
    if (MODE == B2_DKV) {
      const int g = it / w.walk_count;
      hq = w.head_q0 + g;
      q0 = (w.walk_first + it - g * w.walk_count) * kB2Tile;
      k0 = w.own0;
    } else {
      hq = w.head_q0;
      q0 = w.own0;
      k0 = it * kB2Tile;
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < RS; ++s) { mbar_init(bar_res + 8 * s, 1); mbar_init(bar_res_empty + 8 * s, 1); }
    for (int s = 0; s < ST; ++s) { mbar_init(bar_tfull + 8 * s, 1); mbar_init(bar_tempty + 8 * s, 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(bar_sfull + 8 * s, 1); mbar_init(bar_dpfull + 8 * s, 1); }
    mbar_init(bar_sempty, kB2ComputeWarps);
    // P-ready and dS-ready barriers alternate between two by step: the compute warps can finish step g + 1 (whose
    // scores were issued ahead) before the issuer has looked at step g, and a single barrier would then be two phases
    // ahead of the parity the issuer waits for.  Step g + 2 cannot complete before the issuer has passed step g.
    for (int h = 0; h < 2; ++h) {
      mbar_init(bar_pfull + 8 * h, kB2ComputeWarps);
      mbar_init(bar_dsfull + 8 * h, kB2ComputeWarps);
    }
    mbar_init(bar_accfull, 1);
    mbar_init(bar_accempty, kB2ComputeWarps);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == kB2ComputeWarps + 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t sRes = sbase + L::kRes, sStream = sbase + L::kStream;

  if (warp == kB2ComputeWarps) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      uint32_t g = 0, wi = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++wi) {
        Work w;
        get_work(item, w);
        const uint32_t rsl = wi % RS;
        if (!mbar_wait(bar_res_empty + 8 * rsl, ((wi / RS) & 1) ^ 1, abort_flag, status, 60)) break;
        const uint32_t rfull = bar_res + 8 * rsl;
        const uint32_t r0 = sRes + rsl * 2 * L::kTileBytes, r1 = r0 + L::kTileBytes;
        mbar_arrive_expect_tx(rfull, 2 * L::kTileBytes);
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf) {
          if (MODE == B2_DKV) {
            tma_load_4d(r0 + hf * L::kHalf, &tmK, hf * 64, w.head_k, w.own0, w.b, rfull);
            tma_load_4d(r1 + hf * L::kHalf, &tmV, hf * 64, w.head_k, w.own0, w.b, rfull);
          } else {
            tma_load_4d(r0 + hf * L::kHalf, &tmQ, hf * 64, w.head_q0, w.own0, w.b, rfull);
            tma_load_4d(r1 + hf * L::kHalf, &tmdO, hf * 64, w.head_q0, w.own0, w.b, rfull);
          }
        }
        for (int it = 0; it < w.n_it; ++it, ++g) {
          const uint32_t s = g % ST;
          if (!mbar_wait(bar_tempty + 8 * s, ((g / ST) & 1) ^ 1, abort_flag, status, 61)) { ok = false; break; }
          int hq, q0, k0;
          walk_decode(w, it, hq, q0, k0);
          mbar_arrive_expect_tx(bar_tfull + 8 * s, 2 * L::kTileBytes);
          const uint32_t d0 = sStream + s * 2 * L::kTileBytes, d1 = d0 + L::kTileBytes;
#pragma unroll
          for (int hf = 0; hf < D / 64; ++hf) {
            if (MODE == B2_DKV) {
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
  } else if (warp == kB2ComputeWarps + 1) {
    if (lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, D, 0, 1);    // A from TMEM (K-major), B MN-major
      uint32_t res_off = 0;
      // first operand tile of step g's streamed pair / of the resident pair
      auto stream0 = [&](uint32_t g) { return sStream + (g % ST) * 2 * L::kTileBytes; };
      // S (or S^T) and dP (or dP^T) of step g: A and B both K-major [128, D] tiles
      auto issue_s = [&](uint32_t g) {
        const uint32_t t0 = stream0(g), r0 = sRes + res_off;
        const uint32_t a = r0, bq = t0;          // B2_DKV: A = K (resident), B = Q (streamed); B2_DQ: A = Q, B = K
        const uint32_t dst = tmem_base + L::kColS + (SB == 2 ? (g & 1) * 128 : 0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * L::kHalf + (ks & 3) * 32;
          umma_bf16_ss(dst, umma_smem_desc_sw128(a + off, 16, 1024), umma_smem_desc_sw128(bq + off, 16, 1024), idesc_s,
                       ks != 0 ? 1u : 0u);
        }
        umma_commit(bar_sfull + 8 * (SB == 2 ? (g & 1) : 0));
      };
      auto issue_dp = [&](uint32_t g) {
        const uint32_t t1 = stream0(g) + L::kTileBytes, r1 = sRes + res_off + L::kTileBytes;
        // DKV: A = V (resident), B = dO (streamed); DQ: A = dO (resident), B = V (streamed)
        const uint32_t dst = tmem_base + L::kColDp + (DB == 2 ? (g & 1) * 128 : 0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * L::kHalf + (ks & 3) * 32;
          umma_bf16_ss(dst, umma_smem_desc_sw128(r1 + off, 16, 1024), umma_smem_desc_sw128(t1 + off, 16, 1024), idesc_s,
                       ks != 0 ? 1u : 0u);
        }
        umma_commit(bar_dpfull + 8 * (DB == 2 ? (g & 1) : 0));
      };
      // acc += A[TMEM, packed bf16 at columns col0.. (keys / queries 0-63) and col0 + 64.. (64-127)] * B[smem tile, MN-major]
      auto issue_acc = [&](uint32_t acc_col, uint32_t a_col, uint32_t b_tile, bool first) {
#pragma unroll
        for (int ks = 0; ks < kB2Tile / 16; ++ks) {
          const uint32_t a_addr = tmem_base + a_col + (ks < 4 ? ks * 8 : 64 + (ks - 4) * 8);
          umma_bf16_ts(tmem_base + acc_col, a_addr, umma_smem_desc_sw128(b_tile + ks * 2048, L::kHalf, 1024), idesc_acc,
                       (!first || ks != 0) ? 1u : 0u);
        }
      };
      uint32_t g = 0, wi = 0, ai = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++wi) {
        Work w;
        get_work(item, w);
        const uint32_t rsl = wi % RS;
        res_off = rsl * 2 * L::kTileBytes;
        if (!mbar_wait(bar_res + 8 * rsl, (wi / RS) & 1, abort_flag, status, 62)) break;
        if (w.n_it > 0) {
          if (!mbar_wait(bar_tfull + 8 * (g % ST), (g / ST) & 1, abort_flag, status, 63)) break;
          // B2_DQ: the S buffer is free once the compute warps have loaded the previous step's scores.  (B2_DKV: its last
          // reader is the dV product of an earlier step, issued before this point.)
          if (MODE == B2_DQ && g > 0 && !mbar_wait(bar_sempty, (g - 1) & 1, abort_flag, status, 64)) break;
          tc_fence_after();
          issue_s(g);
          issue_dp(g);          // dP buffer of step g: its last reader (step g - DB) was issued long before
          // the compute warps have read out the previous item's accumulators
          if (!mbar_wait(bar_accempty, (ai & 1) ^ 1, abort_flag, status, 65)) break;
        }
        for (int it = 0; it < w.n_it && ok; ++it, ++g) {
          const bool more = it + 1 < w.n_it;
          const uint32_t t0 = stream0(g), t1 = t0 + L::kTileBytes;
          if (MODE == B2_DQ) {
            if (more) {
              if (!mbar_wait(bar_tfull + 8 * ((g + 1) % ST), ((g + 1) / ST) & 1, abort_flag, status, 66)) { ok = false; break; }
              if (!mbar_wait(bar_sempty, g & 1, abort_flag, status, 67)) { ok = false; break; }
              tc_fence_after();
              issue_s(g + 1);
              issue_dp(g + 1);                                   // the other dP buffer: read last by dQ(g - 1), issued
            }
            if (!mbar_wait(bar_dsfull + 8 * (g & 1), (g >> 1) & 1, abort_flag, status, 68)) { ok = false; break; }
            tc_fence_after();
            issue_acc(L::kColAcc0, L::kColDp + (g & 1) * 128, t0, it == 0);          // dQ += dS K
          } else {
            if (more && !mbar_wait(bar_tfull + 8 * ((g + 1) % ST), ((g + 1) / ST) & 1, abort_flag, status, 66)) { ok = false; break; }
            if (more && SB == 2) { tc_fence_after(); issue_s(g + 1); }                // other S^T buffer: free since dV(g - 1)
            if (!mbar_wait(bar_pfull + 8 * (g & 1), (g >> 1) & 1, abort_flag, status, 69)) { ok = false; break; }
            tc_fence_after();
            issue_acc(L::kColAcc1, L::kColS + (SB == 2 ? (g & 1) * 128 : 0), t1, it == 0);   // dV += P^T dO
            if (more && SB == 1) issue_s(g + 1);                                      // reuses the buffer dV(g) just read
            if (!mbar_wait(bar_dsfull + 8 * (g & 1), (g >> 1) & 1, abort_flag, status, 68)) { ok = false; break; }
            tc_fence_after();
            issue_acc(L::kColAcc0, L::kColDp, t0, it == 0);                           // dK += dS^T Q
            if (more) issue_dp(g + 1);                                                // reuses the buffer dK(g) just read
          }
          // every product that reads step g's streamed pair has been issued (step g + 1's products read another stage)
          umma_commit(bar_tempty + 8 * (g % ST));
        }
        if (!ok) break;
        if (w.n_it > 0) {
          umma_commit(bar_accfull);
          ++ai;
        }
        umma_commit(bar_res_empty + 8 * rsl);
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    const int qtr = warp & 3, cg = warp >> 2;              // TMEM lane quarter, column half
    const int row = qtr * 32 + lane;                       // TMEM lane: query (B2_DQ) or key (B2_DKV) inside the tile
    const int ct = threadIdx.x;                            // 0..255 among the compute threads
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    const float sl2 = p.scale * kB2Log2e;
    bool ok = true;
    uint32_t g = 0, ai = 0;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      Work w;
      get_work(item, w);
      const int b = w.b;
      // B2_DQ: this thread's row statistics, fetched one step ahead.  B2_DKV: one value per compute thread of the
      // step's 128 queries (threads 0-127 log-sum-exp, 128-255 delta), staged in shared memory one step ahead.
      auto load_stat_dq = [&](float& lse2, float& dlt) {
        const int q_idx = w.own0 + row;
        lse2 = 0.f; dlt = 0.f;
        if (q_idx < p.seq_q) {
          const long long st = (static_cast<long long>(b) * p.heads + w.head_q0) * p.seq_q + q_idx;
          lse2 = __ldg(p.lse + st) * kB2Log2e;
          dlt = __ldg(p.delta + st);
        }
      };
      auto load_stat_dkv = [&](int it) -> float {
        int hq, q0, k0;
        walk_decode(w, it, hq, q0, k0);
        const int q_idx = q0 + (ct & 127);
        if (q_idx >= p.seq_q) return 0.f;
        const long long st = (static_cast<long long>(b) * p.heads + hq) * p.seq_q + q_idx;
        return ct < 128 ? __ldg(p.lse + st) * kB2Log2e : __ldg(p.delta + st);
      };
      float lse2_row = 0.f, dlt_row = 0.f, stat_next = 0.f;
      if (MODE == B2_DQ) load_stat_dq(lse2_row, dlt_row);
      else if (w.n_it > 0) {
        stats[(g & 1) * 256 + ct] = load_stat_dkv(0);
      }
      for (int it = 0; it < w.n_it && ok; ++it, ++g) {
        int hq, q0, k0;
        walk_decode(w, it, hq, q0, k0);
        const float* st_lse = stats + (g & 1) * 256 + cg * 64;
        const float* st_dlt = st_lse + 128;
        if (MODE == B2_DKV) {
          if (it + 1 < w.n_it) stat_next = load_stat_dkv(it + 1);      // in flight during this step
          b2_bar_compute();                                            // this step's statistics are in shared memory
        }
        // visibility: B2_DQ row = query, columns = keys; B2_DKV row = key, columns = queries
        const int cbase = (MODE == B2_DQ ? k0 : q0) + cg * 64;
        int lim_lo = 0, lim_hi = 0;      // visible columns are [lim_lo, lim_hi]
        if (MODE == B2_DQ) {
          const int q_idx = q0 + row;
          lim_lo = 0;
          lim_hi = q_idx < p.seq_q ? (p.causal ? min(w.kv_len - 1, q_idx + shift) : w.kv_len - 1) : -1;
        } else {
          const int key = k0 + row;
          lim_hi = key < w.kv_len ? p.seq_q - 1 : -1;
          lim_lo = p.causal ? max(0, key - shift) : 0;
        }
        const bool need_mask = cbase < lim_lo || cbase + 63 > lim_hi;
        const uint32_t sb = SB == 2 ? (g & 1) : 0, db = DB == 2 ? (g & 1) : 0;
        const uint32_t t_s = tmem_base + L::kColS + sb * 128 + lane_off + cg * 64;
        const uint32_t t_dp = tmem_base + L::kColDp + db * 128 + lane_off + cg * 64;
        if (!mbar_wait(bar_sfull + 8 * sb, (SB == 2 ? (g >> 1) : g) & 1, abort_flag, status, 70)) { ok = false; break; }
        tc_fence_after();
        // ---- probabilities of this thread's 64 columns (kept in registers as fp32)
        float pr[64];
        {
          uint32_t r[2][16];
          tmem_ld_32x16(t_s, r[0]);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            tmem_ld_wait();
            if (c < 3) tmem_ld_32x16(t_s + (c + 1) * 16, r[(c + 1) & 1]);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int col = c * 16 + i;
              const float l2 = MODE == B2_DQ ? lse2_row : st_lse[col];
              float v = b2_ex2(fmaf(__uint_as_float(r[c & 1][i]), sl2, -l2));
              if (need_mask && (cbase + col < lim_lo || cbase + col > lim_hi)) v = 0.f;
              pr[col] = v;
            }
          }
        }
        if (MODE == B2_DQ) {
          // S is in registers: the next S may overwrite the buffer
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_sempty);
        } else {
          // P^T over this thread's own part of S^T: 64 keys... 64 queries -> 32 packed columns at [cg * 64, cg * 64 + 32)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(pr[c * 32 + 2 * i], pr[c * 32 + 2 * i + 1]);
            tmem_st_32x16(t_s + c * 16, pk);
          }
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_pfull + 8 * (g & 1));
        }
        // ---- dS = P * (dP - delta) -> packed bf16 over this thread's part of the dP buffer
        if (!mbar_wait(bar_dpfull + 8 * db, (DB == 2 ? (g >> 1) : g) & 1, abort_flag, status, 71)) { ok = false; break; }
        tc_fence_after();
        {
          uint32_t r[2][16];
          tmem_ld_32x16(t_dp, r[0]);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            tmem_ld_wait();
            if (c < 3) tmem_ld_32x16(t_dp + (c + 1) * 16, r[(c + 1) & 1]);
            uint32_t pk[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int col = c * 16 + 2 * i;
              const float d0 = MODE == B2_DQ ? dlt_row : st_dlt[col];
              const float d1 = MODE == B2_DQ ? dlt_row : st_dlt[col + 1];
              pk[i] = pack_bf16x2(pr[col] * (__uint_as_float(r[c & 1][2 * i]) - d0),
                                  pr[col + 1] * (__uint_as_float(r[c & 1][2 * i + 1]) - d1));
            }
            // packed columns [8c, 8c + 8) of this thread's part: inside the dP columns already in registers
            asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                         ::"r"(t_dp + c * 8), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]),
                         "r"(pk[6]), "r"(pk[7])
                         : "memory");
          }
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_dsfull + 8 * (g & 1));
        if (MODE == B2_DKV && it + 1 < w.n_it) stats[((g + 1) & 1) * 256 + ct] = stat_next;
      }
      if (!ok) break;

      // ---- read-out: TMEM lane = key (B2_DKV) or query (B2_DQ) row of the owned tile; this column half's share of D
      const bool have = w.n_it > 0;
      if (have && !mbar_wait(bar_accfull, ai & 1, abort_flag, status, 72)) { ok = false; break; }
      tc_fence_after();
      const int r_idx = w.own0 + row;
      const int limit = MODE == B2_DKV ? p.seq_k : p.seq_q;
      const int head_out = MODE == B2_DKV ? w.head_k : w.head_q0;
      constexpr int CW = D / 2;                            // output columns per column half
#pragma unroll
      for (int which = 0; which < (MODE == B2_DKV ? 2 : 1); ++which) {
        const uint32_t tacc = tmem_base + (which == 0 ? L::kColAcc0 : L::kColAcc1);
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
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_accempty);
        ++ai;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kB2ComputeWarps + 1) {
    if (*abort_flag) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace rb

namespace {
const CUtensorMap* b2_map(const void* base, const long long* strides, int seq, int heads, int batch, int D, int* err) {
  long long s[3] = {strides[0] > 0 ? strides[0] : 8, strides[1] > 0 ? strides[1] : D, strides[2] > 0 ? strides[2] : D};
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)heads, (uint64_t)seq, (uint64_t)batch};
  const uint64_t str[3] = {(uint64_t)s[2] * 2, (uint64_t)s[1] * 2, (uint64_t)s[0] * 2};
  const uint32_t box[4] = {64, 1, (uint32_t)rb::kB2Tile, 1};
  return rbhost::get_tmap_4d(base, 2, dims, str, box, 1, err);
}

template <int D, int MODE>
int b2_launch(const CUtensorMap* tq, const CUtensorMap* tk, const CUtensorMap* tv, const CUtensorMap* tdo,
              const rb::B2Params& p, dim3 grid, cudaStream_t stream) {
  auto kern = rb::attn_bwd2_kernel<D, MODE>;
  const int smem = rb::B2Smem<D, MODE>::kTotal + 1024;
  static bool cfg_dev[64] = {false};
  bool& cfg = cfg_dev[rbhost::device_slot()];
  if (!cfg) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    cfg = true;
  }
  kern<<<grid, rb::kB2Threads, smem, stream>>>(*tq, *tk, *tv, *tdo, p, rbhost::status_ptr());
  return static_cast<int>(cudaGetLastError());
}
}  // namespace

// Backward pass, second tcgen05 version (three launches: delta, dK/dV, dQ).  Returns -9 when the problem is outside
// what these kernels take (the caller then uses another backward implementation).
RB_API int rb_attention_bwd_tc2(const RbAttnArgs* a, void* stream_v) {
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
  const CUtensorMap* tq = b2_map(a->q, a->q_strides, a->seq_q, a->heads, a->batch, D, &err);
  const CUtensorMap* tk = b2_map(a->k, a->k_strides, a->seq_k, a->kv_heads, a->batch, D, &err);
  const CUtensorMap* tv = b2_map(a->v, a->v_strides, a->seq_k, a->kv_heads, a->batch, D, &err);
  const CUtensorMap* tdo = b2_map(a->d_o, a->o_strides, a->seq_q, a->heads, a->batch, D, &err);
  if (!tq || !tk || !tv || !tdo) return err ? err : -5;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  int rc = rb_attention_delta_tc(a, stream_v);
  if (rc != 0) return rc;

  rb::B2Params p;
  p.lse = a->lse; p.delta = a->delta;
  p.seq_q = a->seq_q; p.seq_k = a->seq_k; p.heads = a->heads; p.kv_heads = a->kv_heads; p.causal = a->causal;
  p.batch = a->batch;
  p.scale = a->scale;
  p.kv_lens = a->kv_lens;
  p.out0 = reinterpret_cast<__nv_bfloat16*>(a->dk); p.out1 = reinterpret_cast<__nv_bfloat16*>(a->dv);
  p.o0_bs = a->dk_strides[0]; p.o0_rs = a->dk_strides[1]; p.o0_hs = a->dk_strides[2];
  p.o1_bs = a->dv_strides[0]; p.o1_rs = a->dv_strides[1]; p.o1_hs = a->dv_strides[2];
  const int sms = rbhost::device_sm_count();
  const long long kv_items = static_cast<long long>((a->seq_k + rb::kB2Tile - 1) / rb::kB2Tile) * a->kv_heads * a->batch;
  dim3 kvgrid(static_cast<unsigned>(kv_items < sms ? kv_items : sms));
  rc = D == 64 ? b2_launch<64, rb::B2_DKV>(tq, tk, tv, tdo, p, kvgrid, stream)
               : b2_launch<128, rb::B2_DKV>(tq, tk, tv, tdo, p, kvgrid, stream);
  if (rc != 0) return rc;
  p.out0 = reinterpret_cast<__nv_bfloat16*>(a->dq); p.out1 = nullptr;
  p.o0_bs = a->dq_strides[0]; p.o0_rs = a->dq_strides[1]; p.o0_hs = a->dq_strides[2];
  const long long q_items = static_cast<long long>((a->seq_q + rb::kB2Tile - 1) / rb::kB2Tile) * a->heads * a->batch;
  dim3 qgrid(static_cast<unsigned>(q_items < sms ? q_items : sms));
  return D == 64 ? b2_launch<64, rb::B2_DQ>(tq, tk, tv, tdo, p, qgrid, stream)
                 : b2_launch<128, rb::B2_DQ>(tq, tk, tv, tdo, p, qgrid, stream);
}
