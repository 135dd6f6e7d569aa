// Flash attention forward on the 5th-generation tensor cores.
//
// One CTA owns 128 queries of one (batch, head).  Per 128-key tile:
//   S  = Q K^T        tcgen05.mma (SS), accumulator in TMEM (128 fp32 columns)
//   softmax           four warps, one query row per thread: tcgen05.ld S, online max / sum, P (bf16) written to shared
//                     memory in the 128-byte-swizzled layout the MMA reads
//   PV = P V          tcgen05.mma (SS, V read MN-major straight from its [keys, d] layout), accumulator in TMEM
//   O  = O * alpha + PV   in registers (one output row per thread), so TMEM never needs rescaling
// Q, K and V tiles arrive by TMA (4-D tensor maps over the strided [batch, seq, head, dim] views, so a packed QKV
// projection is read in place); K / V are double buffered.  Roles: warps 0-3 softmax + epilogue, warp 4 TMA producer,
// warp 5 MMA issuer.  QK^T of tile j+1 is issued before the softmax of tile j finishes, and with head dim 64 two
// CTAs share an SM, so the tensor cores stay busy while another tile is in its softmax.
//
// Same semantics as the mma.sync kernels in attention.cu (causal alignment to the end of the keys, GQA, log-sum-exp).
#include "attention.h"

#include "rb_common.cuh"

namespace rb {

constexpr int kTcThreads = 192;
constexpr int kTcTile = 128;                 // queries per CTA and keys per tile
constexpr float kTcLog2e = 1.4426950408889634f;

struct TcParams {
  __nv_bfloat16* out;
  float* lse;
  long long o_bs, o_rs, o_hs;
  int seq_q, seq_k, heads, kv_heads, causal;
  float scale;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
struct TcSmem {
  static constexpr int kHalf = kTcTile * 128;                 // one 64-column swizzle atom column: 128 rows x 128 B
  static constexpr int kQBytes = (D / 64) * kHalf;
  static constexpr int kKBytes = (D / 64) * kHalf;            // per stage
  static constexpr int kVBytes = (D / 64) * kHalf;            // per stage
  static constexpr int kPBytes = 2 * kHalf;                   // 128 x 128 bf16
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kQBytes;
  static constexpr int kV = kK + 2 * kKBytes;
  static constexpr int kP = kV + 2 * kVBytes;
  static constexpr int kBar = kP + kPBytes;
  static constexpr int kNumBars = 14;
  static constexpr int kTotal = kBar + kNumBars * 8 + 16;
};

template <int D>
__global__ void __launch_bounds__(kTcThreads)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, TcParams p, unsigned int* status) {
  using L = TcSmem<D>;
  // 1024-byte alignment is requested from the compiler: two CTAs of the head-dim-64 variant only fit on one SM
  // without alignment slack.  A misaligned base (never seen in practice) is reported instead of computing garbage.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t sbase = smem_u32(smem);
  if ((sbase & 1023u) != 0u) {
    if (threadIdx.x == 0) status_set(status, kStatusBadArg, 20);
    return;
  }
  const uint32_t sQ = sbase + L::kQ, sK = sbase + L::kK, sV = sbase + L::kV, sP = sbase + L::kP;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  const uint32_t b0 = smem_u32(bars);
  // barrier indices
  const uint32_t bar_q = b0, bar_kfull = b0 + 8, bar_vfull = b0 + 24, bar_kvempty = b0 + 40, bar_sfull = b0 + 56,
                 bar_sempty = b0 + 64, bar_pfull = b0 + 72, bar_pempty = b0 + 80, bar_pvfull = b0 + 88, bar_pvempty = b0 + 96;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blk = gridDim.x - 1 - blockIdx.x;       // late (long) causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.heads / p.kv_heads);
  const int q0 = m_blk * kTcTile;
  const int shift = p.seq_k - p.seq_q;
  int n_tiles = (p.seq_k + kTcTile - 1) / kTcTile;
  if (p.causal) {
    const int lim = (q0 + kTcTile - 1 + shift) / kTcTile + 1;
    if (lim < n_tiles) n_tiles = lim;
  }
  constexpr uint32_t kTmemCols = 256;                  // S: columns [0,128), PV: [128, 128 + D)

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_kfull + 8 * s, 1);
      mbar_init(bar_vfull + 8 * s, 1);
      mbar_init(bar_kvempty + 8 * s, 1);
    }
    mbar_init(bar_sfull, 1);
    mbar_init(bar_sempty, 4);
    mbar_init(bar_pfull, 4);
    mbar_init(bar_pempty, 1);
    mbar_init(bar_pvfull, 1);
    mbar_init(bar_pvempty, 4);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(tmem_ptr_smem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t tmem_s = tmem_base, tmem_pv = tmem_base + 128;

  if (warp == 4) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      mbar_arrive_expect_tx(bar_q, L::kQBytes);
#pragma unroll
      for (int hf = 0; hf < D / 64; ++hf) tma_load_4d(sQ + hf * L::kHalf, &tmQ, hf * 64, h, q0, b, bar_q);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar_kvempty + 8 * s, ((j >> 1) & 1) ^ 1, abort_flag, status, 21)) break;
        mbar_arrive_expect_tx(bar_kfull + 8 * s, L::kKBytes);
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf)
          tma_load_4d(sK + s * L::kKBytes + hf * L::kHalf, &tmK, hf * 64, hk, j * kTcTile, b, bar_kfull + 8 * s);
        mbar_arrive_expect_tx(bar_vfull + 8 * s, L::kVBytes);
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf)
          tma_load_4d(sV + s * L::kVBytes + hf * L::kHalf, &tmV, hf * 64, hk, j * kTcTile, b, bar_vfull + 8 * s);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, D, 0, 1);        // A = P K-major, B = V MN-major
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(bar_kfull + 8 * s, (j >> 1) & 1, abort_flag, status, 22)) return false;
        if (!mbar_wait(bar_sempty, (j & 1) ^ 1, abort_flag, status, 23)) return false;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * L::kHalf + (ks & 3) * 32;
          umma_bf16_ss(tmem_s, umma_smem_desc_sw128(sQ + off, 16, 1024),
                       umma_smem_desc_sw128(sK + s * L::kKBytes + off, 16, 1024), idesc_qk, ks != 0 ? 1u : 0u);
        }
        umma_commit(bar_sfull);
        return true;
      };
      bool ok = mbar_wait(bar_q, 0, abort_flag, status, 24);
      if (ok && n_tiles > 0) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < n_tiles) {            // S of the next tile overlaps the softmax of this one
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        if (!mbar_wait(bar_pfull, j & 1, abort_flag, status, 25)) break;
        if (!mbar_wait(bar_vfull + 8 * s, (j >> 1) & 1, abort_flag, status, 26)) break;
        if (!mbar_wait(bar_pvempty, (j & 1) ^ 1, abort_flag, status, 27)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < kTcTile / 16; ++ks) {
          const uint64_t da = umma_smem_desc_sw128(sP + (ks >> 2) * L::kHalf + (ks & 3) * 32, 16, 1024);
          // V: 16 key rows of 128 B per step; 64-wide head-dim atoms L::kHalf apart
          const uint64_t db = umma_smem_desc_sw128(sV + s * L::kVBytes + ks * 2048, L::kHalf, 1024);
          umma_bf16_ss(tmem_pv, da, db, idesc_pv, ks != 0 ? 1u : 0u);
        }
        umma_commit(bar_pvfull);
        umma_commit(bar_pempty);
        umma_commit(bar_kvempty + 8 * s);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (one query row per thread)
    const int row = warp * 32 + lane;                     // TMEM lane == query row inside the tile
    const int q_idx = q0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    const float sl2 = p.scale * kTcLog2e;
    float o_acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (!mbar_wait(bar_sfull, j & 1, abort_flag, status, 28)) { ok = false; break; }
      tc_fence_after();
      const int k0 = j * kTcTile;
      const int key_lim = p.causal ? min(p.seq_k - 1, q_idx + shift) : p.seq_k - 1;     // last visible key
      // Only tiles that cross the causal diagonal or the end of the keys need per-element masking.
      const bool need_mask = (k0 + kTcTile - 1 > key_lim);
      // pass 1: row maximum
      float mx = m_run;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_s + lane_off + c * 32, r);
        tmem_ld_wait();
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const int kb = k0 + c * 32 + i;
            m0 = fmaxf(m0, kb <= key_lim ? __uint_as_float(r[i]) : -INFINITY);
            m1 = fmaxf(m1, kb + 1 <= key_lim ? __uint_as_float(r[i + 1]) : -INFINITY);
            m2 = fmaxf(m2, kb + 2 <= key_lim ? __uint_as_float(r[i + 2]) : -INFINITY);
            m3 = fmaxf(m3, kb + 3 <= key_lim ? __uint_as_float(r[i + 3]) : -INFINITY);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            m0 = fmaxf(m0, __uint_as_float(r[i]));
            m1 = fmaxf(m1, __uint_as_float(r[i + 1]));
            m2 = fmaxf(m2, __uint_as_float(r[i + 2]));
            m3 = fmaxf(m3, __uint_as_float(r[i + 3]));
          }
        }
        mx = fmaxf(mx, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
      }
      const float m_safe = mx == -INFINITY ? 0.f : mx;
      const float alpha = ex2_approx((m_run - m_safe) * sl2);
      const float msc = m_safe * sl2;
      m_run = mx;
      // P may be overwritten once the previous PV has read it
      if (!mbar_wait(bar_pempty, (j & 1) ^ 1, abort_flag, status, 29)) { ok = false; break; }
      // pass 2: probabilities -> shared memory (swizzled, K-major A operand of the PV product)
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_s + lane_off + c * 32, r);
        tmem_ld_wait();
        uint32_t packed[16];
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int key = k0 + c * 32 + 2 * i;
            const float p0 = (key <= key_lim) ? ex2_approx(fmaf(__uint_as_float(r[2 * i]), sl2, -msc)) : 0.f;
            const float p1 = (key + 1 <= key_lim) ? ex2_approx(fmaf(__uint_as_float(r[2 * i + 1]), sl2, -msc)) : 0.f;
            rs0 += p0;
            rs1 += p1;
            packed[i] = pack_bf16x2(p0, p1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(r[2 * i]), sl2, -msc));
            const float p1 = ex2_approx(fmaf(__uint_as_float(r[2 * i + 1]), sl2, -msc));
            rs0 += p0;
            rs1 += p1;
            packed[i] = pack_bf16x2(p0, p1);
          }
        }
        // 32 keys = 4 chunks of 16 bytes; key half (c >> 1), chunk index inside the 128-byte row ((c & 1) * 4 + q)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = (c & 1) * 4 + q;
          const uint32_t addr = sP + (c >> 1) * L::kHalf + row * 128 + ((chunk ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(packed[4 * q]), "r"(packed[4 * q + 1]),
                       "r"(packed[4 * q + 2]), "r"(packed[4 * q + 3])
                       : "memory");
        }
      }
      const float rs = rs0 + rs1;
      l_run = l_run * alpha + rs;
      // S has been read twice: the next QK^T may overwrite it; P is complete: PV may start
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar_sempty);
        mbar_arrive(bar_pfull);
      }
      // fold this tile's PV into the running output
      if (!mbar_wait(bar_pvfull, j & 1, abort_flag, status, 30)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_pv + lane_off + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + __uint_as_float(r[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pvempty);
    }
    if (ok && q_idx < p.seq_q) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* op = p.out + b * p.o_bs + h * p.o_hs + static_cast<long long>(q_idx) * p.o_rs;
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        uint4 o;
        o.x = pack_bf16x2(o_acc[c * 8 + 0] * inv, o_acc[c * 8 + 1] * inv);
        o.y = pack_bf16x2(o_acc[c * 8 + 2] * inv, o_acc[c * 8 + 3] * inv);
        o.z = pack_bf16x2(o_acc[c * 8 + 4] * inv, o_acc[c * 8 + 5] * inv);
        o.w = pack_bf16x2(o_acc[c * 8 + 6] * inv, o_acc[c * 8 + 7] * inv);
        reinterpret_cast<uint4*>(op)[c] = o;
      }
      if (p.lse != nullptr)
        p.lse[(static_cast<long long>(b) * p.heads + h) * p.seq_q + q_idx] =
            (m_run == -INFINITY ? 0.f : m_run) * p.scale + logf(fmaxf(l_run, 1e-30f));
    }
  }

  __syncthreads();
  if (warp == 5) {
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
const CUtensorMap* make_map(const void* base, const long long* strides, int seq, int heads, int batch, int D, int* err) {
  // dims innermost first: (d, head, seq, batch); strides in bytes for head, seq, batch
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)heads, (uint64_t)seq, (uint64_t)batch};
  const uint64_t str[3] = {(uint64_t)strides[2] * 2, (uint64_t)strides[1] * 2, (uint64_t)strides[0] * 2};
  const uint32_t box[4] = {64, 1, (uint32_t)rb::kTcTile, 1};
  return rbhost::get_tmap_4d(base, 2, dims, str, box, 1, err);
}
}  // namespace

// Forward pass on the tcgen05 path.  Returns -9 when the problem is outside what this kernel takes (the caller then
// uses rb_attention_fwd).
RB_API int rb_attention_fwd_tc(const RbAttnArgs* a, void* stream_v) {
  if (a->kv_lens) return -9;                 // key-padding lengths: only the second-generation kernels take them
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
  // a tensor-map stride must be non-zero; batch 1 / heads 1 views may carry any stride, give them a valid one
  auto fix = [](const long long* s, long long* out, int D) {
    out[0] = s[0] > 0 ? s[0] : 8; out[1] = s[1] > 0 ? s[1] : D; out[2] = s[2] > 0 ? s[2] : D;
  };
  long long qs[3], ks[3], vs[3];
  fix(a->q_strides, qs, a->head_dim); fix(a->k_strides, ks, a->head_dim); fix(a->v_strides, vs, a->head_dim);
  int err = 0;
  const CUtensorMap* tq = make_map(a->q, qs, a->seq_q, a->heads, a->batch, a->head_dim, &err);
  const CUtensorMap* tk = make_map(a->k, ks, a->seq_k, a->kv_heads, a->batch, a->head_dim, &err);
  const CUtensorMap* tv = make_map(a->v, vs, a->seq_k, a->kv_heads, a->batch, a->head_dim, &err);
  if (!tq || !tk || !tv) return err ? err : -5;
  rb::TcParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(a->o);
  p.lse = a->lse;
  p.o_bs = a->o_strides[0]; p.o_rs = a->o_strides[1]; p.o_hs = a->o_strides[2];
  p.seq_q = a->seq_q; p.seq_k = a->seq_k; p.heads = a->heads; p.kv_heads = a->kv_heads; p.causal = a->causal;
  p.scale = a->scale;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  dim3 grid((a->seq_q + rb::kTcTile - 1) / rb::kTcTile, a->heads, a->batch);
  if (a->head_dim == 64) {
    const int smem = rb::TcSmem<64>::kTotal;
    static bool cfg_dev[64] = {false};
    bool& cfg = cfg_dev[rbhost::device_slot()];
    if (!cfg) { cudaFuncSetAttribute(rb::attn_fwd_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); cfg = true; }
    rb::attn_fwd_tc_kernel<64><<<grid, rb::kTcThreads, smem, stream>>>(*tq, *tk, *tv, p, rbhost::status_ptr());
  } else {
    const int smem = rb::TcSmem<128>::kTotal;
    static bool cfg_dev[64] = {false};
    bool& cfg = cfg_dev[rbhost::device_slot()];
    if (!cfg) { cudaFuncSetAttribute(rb::attn_fwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); cfg = true; }
    rb::attn_fwd_tc_kernel<128><<<grid, rb::kTcThreads, smem, stream>>>(*tq, *tk, *tv, p, rbhost::status_ptr());
  }
  return static_cast<int>(cudaGetLastError());
}
