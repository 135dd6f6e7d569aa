// Flash attention forward, two query tiles per CTA in ping-pong on the 5th-generation tensor cores.
//
// One CTA owns 256 queries of one (batch, head): tile A (rows 0-127) and tile B (rows 128-255).  TMEM (all 512
// columns of the SM) holds S_A, S_B (128 fp32 columns each) and the output accumulators O_A, O_B (head-dim columns
// each).  Per 128-key block j the single MMA-issuing thread runs, in this order,
//     PV(j, A)   O_A += P_A V_j      A operand P read from TMEM (TS form), V_j read MN-major from shared memory
//     QK(j+1, A) S_A  = Q_A K_j+1^T
//     PV(j, B), QK(j+1, B)
// so while softmax warp group A turns S_A into P_A the tensor cores work for tile B and the other way round.
// Softmax (warps 0-3 for A, 4-7 for B, one query row per thread): S is read from TMEM once into registers (the
// producer warp group hands most of its registers to the softmax groups with setmaxnreg), the probabilities are written back as packed bf16 over the first 64 columns of the same S buffer, O stays in TMEM and
// is only rescaled when the running row maximum moved by more than 2^8 (the stale maximum keeps the exponentials
// bounded by 256, exact after the final division by the row sum).  A share of the exponentials can be computed with a
// polynomial on the FMA pipe (template parameter; off by default, see rb_attention_fwd_tc2).  Warp 8 is the TMA producer (Q once, K / V through a ring of stages), warp 9 issues MMAs.
//
// Same semantics as the other forward kernels (causal alignment to the end of the keys, GQA, log-sum-exp output).
// Replaces the reference's materialised-score attention (crates/nn/src/attention.rs:640-836).
#include "attention.h"

#include "rb_common.cuh"

namespace rb {

constexpr int kF2Threads = 384;          // warps 0-7 softmax, 8 TMA, 9 MMA, 10-11 only give their registers away
constexpr int kF2Tile = 128;
constexpr float kF2Log2e = 1.4426950408889634f;
constexpr float kF2RescaleThreshold = 8.f;   // log2 units

struct F2Params {
  __nv_bfloat16* out;
  float* lse;
  long long o_bs, o_rs, o_hs;
  int seq_q, seq_k, heads, kv_heads, causal;
  float scale;
  const int* kv_lens;       // optional [batch]: number of real keys
};

__device__ __forceinline__ float f2_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x on the FMA / integer pipes: round-to-nearest split x = n + f, |f| <= 0.5, degree-4 polynomial for 2^f
// (relative error about 4e-5, well below bf16 rounding), exponent added to the bit pattern.  x must be >= -126.
__device__ __forceinline__ float f2_ex2_poly(float x) {
  x = fmaxf(x, -125.f);
  const float magic = 12582912.f;                     // 1.5 * 2^23: the sum's low mantissa bits hold round(x)
  const float t = x + magic;
  const float n = t - magic;
  const float f = x - n;
  float p = fmaf(f, 0.0096181291f, 0.0555041087f);
  p = fmaf(p, f, 0.2402265070f);
  p = fmaf(p, f, 0.6931471806f);
  p = fmaf(p, f, 1.0f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

// Register reallocation between warp groups (four consecutive warps, all of which must execute the instruction): the
// producer group shrinks to a few registers per thread and the softmax groups grow, so that a whole row of 128 scores
// fits in registers.
// (setmaxnreg_inc / setmaxnreg_dec: rb_common.cuh)

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32_ptr(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

template <int D>
struct F2Smem {
  static constexpr int kStages = D == 64 ? 4 : 2;
  static constexpr int kHalf = kF2Tile * 128;                 // one 64-column swizzle atom: 128 rows x 128 B
  static constexpr int kTileBytes = (D / 64) * kHalf;         // a 128-row tile of Q, K or V
  static constexpr int kQ = 0;                                // two tiles
  static constexpr int kK = kQ + 2 * kTileBytes;
  static constexpr int kV = kK + kStages * kTileBytes;
  static constexpr int kBar = kV + kStages * kTileBytes;
  static constexpr int kNumBars = 2 + 3 * kStages + 6;        // q[2], k_full/v_full/kv_empty[stages], s_full[2], p_full[2], o_ready[2]
  static constexpr int kTotal = kBar + kNumBars * 8 + 16;
};

template <int D, int kPolyEvery>
__global__ void __launch_bounds__(kF2Threads, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, F2Params p, unsigned int* status) {
  using L = F2Smem<D>;
  constexpr int kStages = L::kStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase + L::kQ, sK = sbase + L::kK, sV = sbase + L::kV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  const uint32_t b0 = smem_u32(bars);
  const uint32_t bar_q = b0;                                   // [2]
  const uint32_t bar_kfull = b0 + 16;                          // [kStages]
  const uint32_t bar_vfull = bar_kfull + 8 * kStages;
  const uint32_t bar_kvempty = bar_vfull + 8 * kStages;
  const uint32_t bar_sfull = bar_kvempty + 8 * kStages;        // [2]
  const uint32_t bar_pfull = bar_sfull + 16;                   // [2]
  const uint32_t bar_oready = bar_pfull + 16;                  // [2]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blk = gridDim.x - 1 - blockIdx.x;                // long causal rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.heads / p.kv_heads);
  const int q0 = m_blk * 2 * kF2Tile;
  const int shift = p.seq_k - p.seq_q;
  // keys at positions >= kv_len are padding: never visible, and key blocks that hold only padding are skipped
  const int kv_len = p.kv_lens ? max(0, min(p.seq_k, p.kv_lens[b])) : p.seq_k;
  const int n_all = (kv_len + kF2Tile - 1) / kF2Tile;
  // key blocks seen by tile A and by tile B (0: the tile starts beyond the last query)
  auto blocks_of = [&](int qt) {
    int n = qt < p.seq_q ? n_all : 0;
    if (n > 0 && p.causal) {
      const int lim = (qt + kF2Tile - 1 + shift) / kF2Tile + 1;
      if (lim < n) n = lim;
    }
    return n;
  };
  const int n_a = blocks_of(q0), n_b = blocks_of(q0 + kF2Tile);
  auto n_of = [&](int t) { return t == 0 ? n_a : n_b; };
  const int n_max = n_a > n_b ? n_a : n_b;
  constexpr uint32_t kTmemCols = 512;

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_q + 8 * t, 1);
      mbar_init(bar_sfull + 8 * t, 1);
      mbar_init(bar_pfull + 8 * t, 4);
      mbar_init(bar_oready + 8 * t, 1);
    }
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_kfull + 8 * s, 1);
      mbar_init(bar_vfull + 8 * s, 1);
      mbar_init(bar_kvempty + 8 * s, 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_ptr_smem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp >= 8) {
  setmaxnreg_dec<56>();
  if (warp == 8) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (n_of(t) == 0) continue;
        mbar_arrive_expect_tx(bar_q + 8 * t, L::kTileBytes);
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf)
          tma_load_4d(sQ + t * L::kTileBytes + hf * L::kHalf, &tmQ, hf * 64, h, q0 + t * kF2Tile, b, bar_q + 8 * t);
      }
      for (int j = 0; j < n_max; ++j) {
        const int s = j % kStages, use = j / kStages;
        if (!mbar_wait(bar_kvempty + 8 * s, (use & 1) ^ 1, abort_flag, status, 41)) break;
        mbar_arrive_expect_tx(bar_kfull + 8 * s, L::kTileBytes);
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf)
          tma_load_4d(sK + s * L::kTileBytes + hf * L::kHalf, &tmK, hf * 64, hk, j * kF2Tile, b, bar_kfull + 8 * s);
        mbar_arrive_expect_tx(bar_vfull + 8 * s, L::kTileBytes);
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf)
          tma_load_4d(sV + s * L::kTileBytes + hf * L::kHalf, &tmV, hf * 64, hk, j * kF2Tile, b, bar_vfull + 8 * s);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, D, 0, 1);        // A = P (TMEM, K-major), B = V MN-major
      auto issue_qk = [&](int j, int t) -> bool {
        const int s = j % kStages;
        if (!mbar_wait(bar_kfull + 8 * s, (j / kStages) & 1, abort_flag, status, 42)) return false;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * L::kHalf + (ks & 3) * 32;
          umma_bf16_ss(tmem_base + t * 128, umma_smem_desc_sw128(sQ + t * L::kTileBytes + off, 16, 1024),
                       umma_smem_desc_sw128(sK + s * L::kTileBytes + off, 16, 1024), idesc_qk, ks != 0 ? 1u : 0u);
        }
        umma_commit(bar_sfull + 8 * t);
        return true;
      };
      bool ok = true;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (n_of(t) == 0 || !ok) continue;
        ok = mbar_wait(bar_q + 8 * t, 0, abort_flag, status, 43);
        if (ok) ok = issue_qk(0, t);
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int s = j % kStages;
        if (!mbar_wait(bar_vfull + 8 * s, (j / kStages) & 1, abort_flag, status, 44)) break;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j >= n_of(t) || !ok) continue;
          if (!mbar_wait(bar_pfull + 8 * t, j & 1, abort_flag, status, 45)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tmem_p = tmem_base + t * 128;              // packed bf16 pairs: 8 columns per 16 keys
          const uint32_t tmem_o = tmem_base + 256 + t * 128;
#pragma unroll
          for (int ks = 0; ks < kF2Tile / 16; ++ks) {
            // V: 16 key rows of 128 B per step; 64-wide head-dim atoms L::kHalf apart
            const uint64_t db = umma_smem_desc_sw128(sV + s * L::kTileBytes + ks * 2048, L::kHalf, 1024);
            umma_bf16_ts(tmem_o, tmem_p + ks * 8, db, idesc_pv, (j > 0 || ks != 0) ? 1u : 0u);
          }
          umma_commit(bar_oready + 8 * t);
          if (j + 1 < n_of(t)) ok = issue_qk(j + 1, t);          // overwrites S_t / P_t: ordered behind PV(j, t)
        }
        if (ok) umma_commit(bar_kvempty + 8 * s);               // every MMA that read stage s has been issued
      }
    }
  }
  } else {
    setmaxnreg_inc<224>();
    // ------------------------------------------------------------------ softmax + epilogue, one query row per thread
    const int t = warp >> 2;                                   // query tile of this warp group
    const int wq = warp & 3;                                   // TMEM lane quarter of this warp
    const int row = wq * 32 + lane;
    const int q_idx = q0 + t * kF2Tile + row;
    const uint32_t lane_off = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t tmem_s = tmem_base + t * 128 + lane_off;
    const uint32_t tmem_o = tmem_base + 256 + t * 128 + lane_off;
    const float sl2 = p.scale * kF2Log2e;
    float m_run = -INFINITY, l_run = 0.f;
    const int nt = n_of(t);
    bool ok = true;
    for (int j = 0; j < nt && ok; ++j) {
      if (!mbar_wait(bar_sfull + 8 * t, j & 1, abort_flag, status, 46)) { ok = false; break; }
      tc_fence_after();
      const int k0 = j * kF2Tile;
      const int key_lim = p.causal ? min(kv_len - 1, q_idx + shift) : kv_len - 1;     // last visible key
      const bool need_mask = (k0 + kF2Tile - 1 > key_lim);
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      // maximum over 32 scores (masked keys have been set to -inf)
      auto chunk_max = [&](const uint32_t* v) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(v[i]));
          mx1 = fmaxf(mx1, __uint_as_float(v[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(v[i + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(v[i + 3]));
        }
      };
      // the whole row of 128 scores is read from TMEM once and stays in registers (224 per thread after the
      // reallocation above)
      uint32_t r[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32_ptr(tmem_s + c * 32, r + c * 32);
      tmem_ld_wait();
      if (need_mask) {                               // only blocks that cross the causal diagonal or the end of the keys
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (k0 + i > key_lim) r[i] = 0xff800000u;   // -inf: ignored by the maximum, exp2 gives exactly 0
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) chunk_max(r + c * 32);
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      // Keep the old maximum unless the new one is more than 2^threshold larger: exponentials stay <= 2^threshold.
      const bool grow = (mx > m_run) && ((mx - m_run) * sl2 > kF2RescaleThreshold || m_run == -INFINITY);
      float alpha = 1.f;
      if (grow) {
        alpha = (m_run == -INFINITY) ? 0.f : f2_ex2((m_run - mx) * sl2);
        m_run = mx;
        l_run *= alpha;
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // O_t holds the sum over blocks 0..j-1 once PV(j-1, t) has completed; PV(j, t) cannot start before P below.
        if (!mbar_wait(bar_oready + 8 * t, (j - 1) & 1, abort_flag, status, 47)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32_ptr(tmem_o + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(tmem_o + c * 32, o);
        }
        tmem_st_wait();
      }
      const float msc = (m_run == -INFINITY ? 0.f : m_run) * sl2;
      float rs0 = 0.f, rs1 = 0.f;
      constexpr int kDiv = kPolyEvery > 0 ? kPolyEvery : 1;
      // 32 scores starting at key kb -> probabilities, 16 packed bf16 pairs (chunk index c selects the polynomial share)
      auto chunk_exp = [&](const uint32_t* v, int kb, int c, uint32_t* packed) {
#pragma unroll
        for (int ii = 0; ii < 16; ++ii) {
          const int i = c * 16 + ii;
          const float x0 = fmaf(__uint_as_float(v[2 * ii]), sl2, -msc);
          const float x1 = fmaf(__uint_as_float(v[2 * ii + 1]), sl2, -msc);
          float p0, p1;
          if (kPolyEvery > 0 && (i % kDiv) == kDiv - 1) {
            p0 = f2_ex2_poly(x0);
            p1 = f2_ex2_poly(x1);
          } else {
            p0 = f2_ex2(x0);
            p1 = f2_ex2(x1);
          }
          if (kPolyEvery > 0 && need_mask) {           // the polynomial clamps its argument: zero masked keys explicitly
            if (kb + 2 * ii > key_lim) p0 = 0.f;
            if (kb + 2 * ii + 1 > key_lim) p1 = 0.f;
          }
          rs0 += p0;
          rs1 += p1;
          packed[ii] = pack_bf16x2(p0, p1);
        }
      };
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t packed[16];
        chunk_exp(r + c * 32, k0 + c * 32, c, packed);
        // columns [16c, 16c + 16) of the score buffer: every score is already in registers
        tmem_st_32x16(tmem_s + c * 16, packed);
      }
      l_run += rs0 + rs1;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pfull + 8 * t);
    }
    if (ok && nt > 0) ok = mbar_wait(bar_oready + 8 * t, (nt - 1) & 1, abort_flag, status, 48);
    if (nt == 0 && q_idx < p.seq_q && q0 + t * kF2Tile < p.seq_q) {
      // no visible key at all (every key of this batch entry is padding): the output row is zero
      __nv_bfloat16* op = p.out + b * p.o_bs + h * p.o_hs + static_cast<long long>(q_idx) * p.o_rs;
#pragma unroll
      for (int c = 0; c < D / 8; ++c) reinterpret_cast<uint4*>(op)[c] = make_uint4(0u, 0u, 0u, 0u);
      if (p.lse != nullptr) p.lse[(static_cast<long long>(b) * p.heads + h) * p.seq_q + q_idx] = 0.f;
    }
    if (ok && nt > 0) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* op = p.out + b * p.o_bs + h * p.o_hs + static_cast<long long>(q_idx) * p.o_rs;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32_ptr(tmem_o + c * 32, o);
        tmem_ld_wait();
        if (q_idx < p.seq_q) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[g * 8 + 0]) * inv, __uint_as_float(o[g * 8 + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv);
            reinterpret_cast<uint4*>(op)[c * 4 + g] = v;
          }
        }
      }
      if (p.lse != nullptr && q_idx < p.seq_q)
        p.lse[(static_cast<long long>(b) * p.heads + h) * p.seq_q + q_idx] =
            (m_run == -INFINITY ? 0.f : m_run) * p.scale + logf(fmaxf(l_run, 1e-30f));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    if (*abort_flag) {
      // a wait gave up: let copies and MMAs in flight land before the accumulators are released
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace rb

namespace {
const CUtensorMap* f2_make_map(const void* base, const long long* strides, int seq, int heads, int batch, int D, int* err) {
  // dims innermost first: (d, head, seq, batch); strides in bytes for head, seq, batch
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)heads, (uint64_t)seq, (uint64_t)batch};
  const uint64_t str[3] = {(uint64_t)strides[2] * 2, (uint64_t)strides[1] * 2, (uint64_t)strides[0] * 2};
  const uint32_t box[4] = {64, 1, (uint32_t)rb::kF2Tile, 1};
  return rbhost::get_tmap_4d(base, 2, dims, str, box, 1, err);
}

template <int D, int P>
int f2_launch(const CUtensorMap* tq, const CUtensorMap* tk, const CUtensorMap* tv, const rb::F2Params& p, dim3 grid,
              cudaStream_t stream) {
  auto kern = rb::attn_fwd2_kernel<D, P>;
  const int smem = rb::F2Smem<D>::kTotal + 1024;
  static bool cfg_dev[64] = {false};
  bool& cfg = cfg_dev[rbhost::device_slot()];
  if (!cfg) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    cfg = true;
  }
  kern<<<grid, rb::kF2Threads, smem, stream>>>(*tq, *tk, *tv, p, rbhost::status_ptr());
  return static_cast<int>(cudaGetLastError());
}
}  // namespace

// Forward pass with two query tiles per CTA.  `poly_every`: 0 = every exponential on the special-function unit,
// 4 = every fourth pair of keys on the FMA-pipe polynomial (measured slower on B200 at both head dims: 218 us against
// 191 us for batch 32 x 12 heads x 1024 x 64; kept for parts whose special-function unit is the limit).  Returns -9 for problems this kernel does not
// take (the caller then uses another forward kernel).
RB_API int rb_attention_fwd_tc2(const RbAttnArgs* a, int poly_every, void* stream_v) {
  if (a->batch <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads) return -1;
  if (a->head_dim != 64 && a->head_dim != 128) return -9;
  if (a->seq_q <= 0 || a->seq_k <= 0 || (a->causal && a->seq_q > a->seq_k)) return -1;
  const void* ptrs[4] = {a->q, a->k, a->v, a->o};
  for (int i = 0; i < 4; ++i)
    if (!ptrs[i] || (reinterpret_cast<uintptr_t>(ptrs[i]) & 15)) return -9;
  const long long* strs[4] = {a->q_strides, a->k_strides, a->v_strides, a->o_strides};
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 3; ++j)
      if (strs[i][j] % 8) return -9;            // TMA strides are multiples of 16 bytes
  auto fix = [](const long long* s, long long* out, int D) {
    out[0] = s[0] > 0 ? s[0] : 8; out[1] = s[1] > 0 ? s[1] : D; out[2] = s[2] > 0 ? s[2] : D;
  };
  long long qs[3], ks[3], vs[3];
  fix(a->q_strides, qs, a->head_dim); fix(a->k_strides, ks, a->head_dim); fix(a->v_strides, vs, a->head_dim);
  int err = 0;
  const CUtensorMap* tq = f2_make_map(a->q, qs, a->seq_q, a->heads, a->batch, a->head_dim, &err);
  const CUtensorMap* tk = f2_make_map(a->k, ks, a->seq_k, a->kv_heads, a->batch, a->head_dim, &err);
  const CUtensorMap* tv = f2_make_map(a->v, vs, a->seq_k, a->kv_heads, a->batch, a->head_dim, &err);
  if (!tq || !tk || !tv) return err ? err : -5;
  rb::F2Params p;
  p.out = reinterpret_cast<__nv_bfloat16*>(a->o);
  p.lse = a->lse;
  p.o_bs = a->o_strides[0]; p.o_rs = a->o_strides[1]; p.o_hs = a->o_strides[2];
  p.seq_q = a->seq_q; p.seq_k = a->seq_k; p.heads = a->heads; p.kv_heads = a->kv_heads; p.causal = a->causal;
  p.scale = a->scale;
  p.kv_lens = a->kv_lens;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  dim3 grid((a->seq_q + 2 * rb::kF2Tile - 1) / (2 * rb::kF2Tile), a->heads, a->batch);
  if (a->head_dim == 64) {
    switch (poly_every) {
      case 0: return f2_launch<64, 0>(tq, tk, tv, p, grid, stream);
      case 4: return f2_launch<64, 4>(tq, tk, tv, p, grid, stream);
      default: return -1;
    }
  }
  switch (poly_every) {
    case 0: return f2_launch<128, 0>(tq, tk, tv, p, grid, stream);
    case 4: return f2_launch<128, 4>(tq, tk, tv, p, grid, stream);
    default: return -1;
  }
}
