// Flash attention forward and backward (causal or full, MHA / GQA / MQA, head dim 64 or 128).
//
// Tiled online-softmax attention with O(S) memory: scores never leave the SM.  Forward keeps the
// log-sum-exp per row; backward recomputes probabilities from it and runs as two kernels (one owns a
// K/V tile and produces dK, dV; one owns a Q tile and produces dQ), so no floating-point atomics are
// needed and gradients are bit-reproducible.  Tensors are addressed through (batch, row, head)
// strides, so the packed [tokens, 3*d_model] output of a fused QKV projection is consumed in place
// and gradients are written in the same packed layout.
//
// Tensor-core path in this file: mma.sync m16n8k16 bf16 with ldmatrix-fed fragments and cp.async
// double buffering.
//
// Replaces the reference's attention, which materialises the S x S score matrix, never applies its
// causal mask and soft-maxes over all flattened scores (crates/nn/src/attention.rs:105-144,750-835;
// crates/nn/src/tape_transformer.rs:104-132; crates/candle-backend/src/lib.rs:351-397).
#include "attention.h"

#include "rb_common.cuh"

namespace rb {

constexpr int kAttnThreads = 128;
constexpr int kTile = 64;
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
  const __nv_bfloat16 *q, *k, *v, *o, *d_o;
  __nv_bfloat16 *out, *dq, *dk, *dv;
  float *lse, *delta;
  long long q_bs, q_rs, q_hs;      // element strides: batch, row (token), head
  long long k_bs, k_rs, k_hs;
  long long v_bs, v_rs, v_hs;
  long long o_bs, o_rs, o_hs;      // o / out / d_o share strides
  long long dq_bs, dq_rs, dq_hs;
  long long dk_bs, dk_rs, dk_hs;
  long long dv_bs, dv_rs, dv_hs;
  int seq_q, seq_k, heads, kv_heads, causal;
  float scale;
};

// ------------------------------------------------------------------------------------------ smem tiles
template <int D>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
  return base + row * (D * 2) + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Loads rows [row0, row0+64) of a [rows, D] strided matrix into a swizzled smem tile; rows >= nrows are zero-filled.
template <int D>
__device__ __forceinline__ void load_tile(uint32_t smem, const __nv_bfloat16* g, long long row_stride, int row0, int nrows) {
  constexpr int kChunks = D / 8;
#pragma unroll
  for (int i = threadIdx.x; i < kTile * kChunks; i += kAttnThreads) {
    const int r = i / kChunks, c = i % kChunks;
    const bool valid = (row0 + r) < nrows;
    const __nv_bfloat16* src = g + static_cast<long long>(valid ? row0 + r : 0) * row_stride + c * 8;
    cp_async16(tile_addr<D>(smem, r, c), src, valid);
  }
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A fragment (16 rows x 16 k) of a row-major tile
template <int D>
__device__ __forceinline__ void load_a(uint32_t smem, int row0, int k0, uint32_t (&a)[4]) {
  const int lane = threadIdx.x & 31;
  ldsm_x4(tile_addr<D>(smem, row0 + (lane & 15), (k0 >> 3) + (lane >> 4)), a[0], a[1], a[2], a[3]);
}
// B fragments for 16 n x 16 k where the tile is stored [n][k]: (b[0],b[1]) -> n 0..7, (b[2],b[3]) -> n 8..15
template <int D>
__device__ __forceinline__ void load_b_nk(uint32_t smem, int n0, int k0, uint32_t (&b)[4]) {
  const int lane = threadIdx.x & 31;
  const int mi = lane >> 3;
  ldsm_x4(tile_addr<D>(smem, n0 + ((mi >> 1) << 3) + (lane & 7), (k0 >> 3) + (mi & 1)), b[0], b[1], b[2], b[3]);
}
// B fragments for 16 k x 16 n where the tile is stored [k][n]: (b[0],b[1]) -> n 0..7, (b[2],b[3]) -> n 8..15
template <int D>
__device__ __forceinline__ void load_b_kn(uint32_t smem, int k0, int n0, uint32_t (&b)[4]) {
  const int lane = threadIdx.x & 31;
  const int mi = lane >> 3;
  ldsm_x4_t(tile_addr<D>(smem, k0 + ((mi & 1) << 3) + (lane & 7), (n0 >> 3) + (mi >> 1)), b[0], b[1], b[2], b[3]);
}

// acc[16 x 64] = A(16 x D from a_smem rows a_row0..) * B^T with B stored [64][D]
template <int D>
__device__ __forceinline__ void gemm_rows_nk(float (&acc)[8][4], uint32_t a_smem, int a_row0, uint32_t b_smem) {
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    load_a<D>(a_smem, a_row0, kk * 16, a);
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t b[4];
      load_b_nk<D>(b_smem, np * 16, kk * 16, b);
      mma_bf16(acc[2 * np], a, b[0], b[1]);
      mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// out[16 x D] += P(16 x 64, from accumulator-layout registers) * B with B stored [64][D]
template <int D>
__device__ __forceinline__ void gemm_p_kn(float (&out)[D / 8][4], const float (&p)[8][4], uint32_t b_smem) {
#pragma unroll
  for (int kt = 0; kt < 4; ++kt) {
    uint32_t a[4];
    a[0] = pack_bf16x2(p[2 * kt][0], p[2 * kt][1]);
    a[1] = pack_bf16x2(p[2 * kt][2], p[2 * kt][3]);
    a[2] = pack_bf16x2(p[2 * kt + 1][0], p[2 * kt + 1][1]);
    a[3] = pack_bf16x2(p[2 * kt + 1][2], p[2 * kt + 1][3]);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t b[4];
      load_b_kn<D>(b_smem, kt * 16, dp * 16, b);
      mma_bf16(out[2 * dp], a, b[0], b[1]);
      mma_bf16(out[2 * dp + 1], a, b[2], b[3]);
    }
  }
}

// Writes a warp's 16 x D fp32 accumulator as bf16 into rows [row0, row0+16) of a swizzled tile.
template <int D>
__device__ __forceinline__ void acc_to_tile(uint32_t smem, int row0, const float (&acc)[D / 8][4], float mul0, float mul1) {
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    const uint32_t lo = pack_bf16x2(acc[nt][0] * mul0, acc[nt][1] * mul0);
    const uint32_t hi = pack_bf16x2(acc[nt][2] * mul1, acc[nt][3] * mul1);
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile_addr<D>(smem, row0 + g, nt) + t * 4), "r"(lo) : "memory");
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile_addr<D>(smem, row0 + g + 8, nt) + t * 4), "r"(hi) : "memory");
  }
}
// Copies a swizzled 64 x D tile to global rows [row0, ...), skipping rows >= nrows.
template <int D>
__device__ __forceinline__ void store_tile(uint32_t smem, __nv_bfloat16* g, long long row_stride, int row0, int nrows) {
  constexpr int kChunks = D / 8;
#pragma unroll
  for (int i = threadIdx.x; i < kTile * kChunks; i += kAttnThreads) {
    const int r = i / kChunks, c = i % kChunks;
    if (row0 + r < nrows) {
      uint4 v;
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(tile_addr<D>(smem, r, c)));
      *reinterpret_cast<uint4*>(g + static_cast<long long>(row0 + r) * row_stride + c * 8) = v;
    }
  }
}

// ------------------------------------------------------------------------------------------ forward
template <int D>
__global__ void __launch_bounds__(kAttnThreads)
attn_fwd_kernel(AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int kTileBytes = kTile * D * 2;
  const uint32_t sQ = smem_u32(smem_raw);
  const uint32_t sK = sQ + kTileBytes;           // 2 buffers
  const uint32_t sV = sK + 2 * kTileBytes;       // 2 buffers

  const int m_blk = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.heads / p.kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int m0 = m_blk * kTile;

  const __nv_bfloat16* qg = p.q + b * p.q_bs + h * p.q_hs;
  const __nv_bfloat16* kg = p.k + b * p.k_bs + hk * p.k_hs;
  const __nv_bfloat16* vg = p.v + b * p.v_bs + hk * p.v_hs;

  // with a causal mask and seq_q <= seq_k the queries are aligned to the END of the keys
  const int shift = p.seq_k - p.seq_q;
  int n_tiles = (p.seq_k + kTile - 1) / kTile;
  if (p.causal) {
    const int last_key = m0 + kTile - 1 + shift;
    const int lim = last_key / kTile + 1;
    if (lim < n_tiles) n_tiles = lim;
  }

  load_tile<D>(sQ, qg, p.q_rs, m0, p.seq_q);
  load_tile<D>(sK, kg, p.k_rs, 0, p.seq_k);
  load_tile<D>(sV, vg, p.v_rs, 0, p.seq_k);
  cp_async_commit();

  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sl2 = p.scale * kLog2e;
  const int q_idx0 = m0 + warp * 16 + g + shift;   // key index limit for row g; row g+8 adds 8

  for (int j = 0; j < n_tiles; ++j) {
    const int buf = j & 1;
    if (j + 1 < n_tiles) {
      load_tile<D>(sK + (buf ^ 1) * kTileBytes, kg, p.k_rs, (j + 1) * kTile, p.seq_k);
      load_tile<D>(sV + (buf ^ 1) * kTileBytes, vg, p.v_rs, (j + 1) * kTile, p.seq_k);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) s[i][jj] = 0.f;
    gemm_rows_nk<D>(s, sQ, warp * 16, sK + buf * kTileBytes);

    const int k0 = j * kTile;
    const bool need_mask = (k0 + kTile > p.seq_k) || (p.causal && (k0 + kTile - 1 > m0 + warp * 16 + shift));
    if (need_mask) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = k0 + nt * 8 + 2 * t + (e & 1);
          const int lim = q_idx0 + ((e >> 1) << 3);
          if (key >= p.seq_k || (p.causal && key > lim)) s[nt][e] = -INFINITY;
        }
    }
    float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float alpha[2], msc[2], rs[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float m_safe = mx[r] == -INFINITY ? 0.f : mx[r];
      alpha[r] = exp2f((m_run[r] - m_safe) * sl2);   // m_run = -inf -> 0
      msc[r] = m_safe * sl2;
      m_run[r] = mx[r];
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      s[nt][0] = exp2f(s[nt][0] * sl2 - msc[0]);
      s[nt][1] = exp2f(s[nt][1] * sl2 - msc[0]);
      s[nt][2] = exp2f(s[nt][2] * sl2 - msc[1]);
      s[nt][3] = exp2f(s[nt][3] * sl2 - msc[1]);
      rs[0] += s[nt][0] + s[nt][1];
      rs[1] += s[nt][2] + s[nt][3];
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + rs[r];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o_acc[i][0] *= alpha[0]; o_acc[i][1] *= alpha[0];
      o_acc[i][2] *= alpha[1]; o_acc[i][3] *= alpha[1];
    }
    gemm_p_kn<D>(o_acc, s, sV + buf * kTileBytes);
    __syncthreads();
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
  const float inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
  acc_to_tile<D>(sQ, warp * 16, o_acc, inv0, inv1);   // each warp overwrites only its own Q rows
  if (p.lse != nullptr && t == 0) {
    const long long base = (static_cast<long long>(b) * p.heads + h) * p.seq_q;
    const int r0 = m0 + warp * 16 + g;
    if (r0 < p.seq_q) p.lse[base + r0] = (m_run[0] == -INFINITY ? 0.f : m_run[0]) * p.scale + logf(fmaxf(l_run[0], 1e-30f));
    if (r0 + 8 < p.seq_q) p.lse[base + r0 + 8] = (m_run[1] == -INFINITY ? 0.f : m_run[1]) * p.scale + logf(fmaxf(l_run[1], 1e-30f));
  }
  __syncthreads();
  store_tile<D>(sQ, p.out + b * p.o_bs + h * p.o_hs, p.o_rs, m0, p.seq_q);
}

// ------------------------------------------------------------------------------------------ backward
// delta[b, h, s] = sum_d o * d_o
template <int D>
__global__ void __launch_bounds__(128) attn_delta_kernel(AttnParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * 4 + warp;   // over b * heads * seq_q
  const long long total = static_cast<long long>(p.heads) * p.seq_q;
  const int b = blockIdx.y;
  if (row >= total) return;
  const int h = static_cast<int>(row / p.seq_q);
  const int s = static_cast<int>(row - static_cast<long long>(h) * p.seq_q);
  const __nv_bfloat16* o = p.o + b * p.o_bs + h * p.o_hs + static_cast<long long>(s) * p.o_rs;
  const __nv_bfloat16* d = p.d_o + b * p.o_bs + h * p.o_hs + static_cast<long long>(s) * p.o_rs;
  float acc = 0.f;
  for (int c = lane * 2; c < D; c += 64) {
    const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(o + c));
    const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(d + c));
    acc += a.x * g.x + a.y * g.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) p.delta[(static_cast<long long>(b) * p.heads + h) * p.seq_q + s] = acc;
}

// One CTA owns 64 keys of one KV head: dK, dV.
template <int D>
__global__ void __launch_bounds__(kAttnThreads)
attn_bwd_dkv_kernel(AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int kTileBytes = kTile * D * 2;
  const uint32_t sK = smem_u32(smem_raw);
  const uint32_t sV = sK + kTileBytes;
  const uint32_t sQ = sV + kTileBytes;            // 2 buffers
  const uint32_t sdO = sQ + 2 * kTileBytes;       // 2 buffers
  float* s_lse = reinterpret_cast<float*>(smem_raw + 6 * kTileBytes);   // [2][64]
  float* s_delta = s_lse + 2 * kTile;                                   // [2][64]

  const int n_blk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = n_blk * kTile;
  const int group = p.heads / p.kv_heads;
  const int shift = p.seq_k - p.seq_q;
  const float sl2 = p.scale * kLog2e;

  const __nv_bfloat16* kg = p.k + b * p.k_bs + hk * p.k_hs;
  const __nv_bfloat16* vg = p.v + b * p.v_bs + hk * p.v_hs;
  load_tile<D>(sK, kg, p.k_rs, n0, p.seq_k);
  load_tile<D>(sV, vg, p.v_rs, n0, p.seq_k);
  cp_async_commit();

  const int num_q_tiles = (p.seq_q + kTile - 1) / kTile;
  int first_q = 0;
  if (p.causal) {
    const int fq = n0 - shift;           // first query that can see key n0
    first_q = fq > 0 ? fq / kTile : 0;
  }
  const int per_head = num_q_tiles - first_q;
  const int total_iters = per_head > 0 ? per_head * group : 0;

  float dk_acc[D / 8][4], dv_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { dk_acc[i][j] = 0.f; dv_acc[i][j] = 0.f; }

  auto issue = [&](int it, int buf) {
    const int hq = hk * group + it / per_head;
    const int qt = first_q + it % per_head;
    const __nv_bfloat16* qg = p.q + b * p.q_bs + hq * p.q_hs;
    const __nv_bfloat16* dog = p.d_o + b * p.o_bs + hq * p.o_hs;
    load_tile<D>(sQ + buf * kTileBytes, qg, p.q_rs, qt * kTile, p.seq_q);
    load_tile<D>(sdO + buf * kTileBytes, dog, p.o_rs, qt * kTile, p.seq_q);
    if (threadIdx.x < kTile) {
      const int r = qt * kTile + threadIdx.x;
      const long long base = (static_cast<long long>(b) * p.heads + hq) * p.seq_q;
      s_lse[buf * kTile + threadIdx.x] = r < p.seq_q ? p.lse[base + r] : INFINITY;   // +inf -> probability 0
      s_delta[buf * kTile + threadIdx.x] = r < p.seq_q ? p.delta[base + r] : 0.f;
    }
  };

  if (total_iters > 0) { issue(0, 0); }
  cp_async_commit();

  for (int it = 0; it < total_iters; ++it) {
    const int buf = it & 1;
    if (it + 1 < total_iters) {
      issue(it + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int qt = first_q + it % per_head;
    const int q0 = qt * kTile;

    // S^T (16 keys x 64 queries) = K_w Q^T
    float st[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) st[i][j] = 0.f;
    gemm_rows_nk<D>(st, sK, warp * 16, sQ + buf * kTileBytes);
    // dP^T = V_w dO^T
    float dpt[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) dpt[i][j] = 0.f;
    gemm_rows_nk<D>(dpt, sV, warp * 16, sdO + buf * kTileBytes);

    const float* lse_b = s_lse + buf * kTile;
    const float* del_b = s_delta + buf * kTile;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int qc = nt * 8 + 2 * t + (e & 1);          // query column inside the tile
        const int key = n0 + warp * 16 + g + ((e >> 1) << 3);
        const int qi = q0 + qc;
        float pr = exp2f(st[nt][e] * sl2 - lse_b[qc] * kLog2e);
        if (key >= p.seq_k || (p.causal && key > qi + shift)) pr = 0.f;
        st[nt][e] = pr;
        dpt[nt][e] = pr * (dpt[nt][e] - del_b[qc]);
      }
    gemm_p_kn<D>(dv_acc, st, sdO + buf * kTileBytes);    // dV += P^T dO
    gemm_p_kn<D>(dk_acc, dpt, sQ + buf * kTileBytes);    // dK += dS^T Q
    __syncthreads();
  }

  cp_async_wait<0>();
  __syncthreads();
  // stage through the (now idle) Q / dO buffers and write out coalesced
  acc_to_tile<D>(sQ, warp * 16, dk_acc, p.scale, p.scale);
  acc_to_tile<D>(sdO, warp * 16, dv_acc, 1.f, 1.f);
  __syncthreads();
  store_tile<D>(sQ, p.dk + b * p.dk_bs + hk * p.dk_hs, p.dk_rs, n0, p.seq_k);
  store_tile<D>(sdO, p.dv + b * p.dv_bs + hk * p.dv_hs, p.dv_rs, n0, p.seq_k);
}

// One CTA owns 64 queries of one head: dQ.
template <int D>
__global__ void __launch_bounds__(kAttnThreads)
attn_bwd_dq_kernel(AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int kTileBytes = kTile * D * 2;
  const uint32_t sQ = smem_u32(smem_raw);
  const uint32_t sdO = sQ + kTileBytes;
  const uint32_t sK = sdO + kTileBytes;           // 2 buffers
  const uint32_t sV = sK + 2 * kTileBytes;        // 2 buffers

  const int m_blk = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.heads / p.kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int m0 = m_blk * kTile;
  const int shift = p.seq_k - p.seq_q;
  const float sl2 = p.scale * kLog2e;

  const __nv_bfloat16* qg = p.q + b * p.q_bs + h * p.q_hs;
  const __nv_bfloat16* dog = p.d_o + b * p.o_bs + h * p.o_hs;
  const __nv_bfloat16* kg = p.k + b * p.k_bs + hk * p.k_hs;
  const __nv_bfloat16* vg = p.v + b * p.v_bs + hk * p.v_hs;

  int n_tiles = (p.seq_k + kTile - 1) / kTile;
  if (p.causal) {
    const int lim = (m0 + kTile - 1 + shift) / kTile + 1;
    if (lim < n_tiles) n_tiles = lim;
  }
  load_tile<D>(sQ, qg, p.q_rs, m0, p.seq_q);
  load_tile<D>(sdO, dog, p.o_rs, m0, p.seq_q);
  load_tile<D>(sK, kg, p.k_rs, 0, p.seq_k);
  load_tile<D>(sV, vg, p.v_rs, 0, p.seq_k);
  cp_async_commit();

  const long long base = (static_cast<long long>(b) * p.heads + h) * p.seq_q;
  const int r0 = m0 + warp * 16 + g;
  float lse_r[2], del_r[2];
  lse_r[0] = r0 < p.seq_q ? p.lse[base + r0] * kLog2e : INFINITY;
  lse_r[1] = r0 + 8 < p.seq_q ? p.lse[base + r0 + 8] * kLog2e : INFINITY;
  del_r[0] = r0 < p.seq_q ? p.delta[base + r0] : 0.f;
  del_r[1] = r0 + 8 < p.seq_q ? p.delta[base + r0 + 8] : 0.f;

  float dq_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) dq_acc[i][j] = 0.f;

  for (int j = 0; j < n_tiles; ++j) {
    const int buf = j & 1;
    if (j + 1 < n_tiles) {
      load_tile<D>(sK + (buf ^ 1) * kTileBytes, kg, p.k_rs, (j + 1) * kTile, p.seq_k);
      load_tile<D>(sV + (buf ^ 1) * kTileBytes, vg, p.v_rs, (j + 1) * kTile, p.seq_k);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float s[8][4], dp[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) { s[i][jj] = 0.f; dp[i][jj] = 0.f; }
    gemm_rows_nk<D>(s, sQ, warp * 16, sK + buf * kTileBytes);
    gemm_rows_nk<D>(dp, sdO, warp * 16, sV + buf * kTileBytes);
    const int k0 = j * kTile;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = k0 + nt * 8 + 2 * t + (e & 1);
        const int r = e >> 1;
        const int qi = r0 + (r << 3);
        float pr = exp2f(s[nt][e] * sl2 - lse_r[r]);
        if (key >= p.seq_k || (p.causal && key > qi + shift)) pr = 0.f;
        s[nt][e] = pr * (dp[nt][e] - del_r[r]);
      }
    gemm_p_kn<D>(dq_acc, s, sK + buf * kTileBytes);   // dQ += dS K
    __syncthreads();
  }
  acc_to_tile<D>(sQ, warp * 16, dq_acc, p.scale, p.scale);
  __syncthreads();
  store_tile<D>(sQ, p.dq + b * p.dq_bs + h * p.dq_hs, p.dq_rs, m0, p.seq_q);
}

}  // namespace rb

namespace {
bool fill_params(const RbAttnArgs* a, rb::AttnParams& p) {
  if (a->batch <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads != 0) return false;
  if (a->seq_q <= 0 || a->seq_k <= 0 || (a->head_dim != 64 && a->head_dim != 128)) return false;
  if (a->causal && a->seq_q > a->seq_k) return false;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a->q); p.k = reinterpret_cast<const __nv_bfloat16*>(a->k);
  p.v = reinterpret_cast<const __nv_bfloat16*>(a->v); p.o = reinterpret_cast<const __nv_bfloat16*>(a->o);
  p.d_o = reinterpret_cast<const __nv_bfloat16*>(a->d_o); p.out = reinterpret_cast<__nv_bfloat16*>(a->o);
  p.dq = reinterpret_cast<__nv_bfloat16*>(a->dq); p.dk = reinterpret_cast<__nv_bfloat16*>(a->dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(a->dv);
  p.lse = a->lse; p.delta = a->delta;
  p.q_bs = a->q_strides[0]; p.q_rs = a->q_strides[1]; p.q_hs = a->q_strides[2];
  p.k_bs = a->k_strides[0]; p.k_rs = a->k_strides[1]; p.k_hs = a->k_strides[2];
  p.v_bs = a->v_strides[0]; p.v_rs = a->v_strides[1]; p.v_hs = a->v_strides[2];
  p.o_bs = a->o_strides[0]; p.o_rs = a->o_strides[1]; p.o_hs = a->o_strides[2];
  p.dq_bs = a->dq_strides[0]; p.dq_rs = a->dq_strides[1]; p.dq_hs = a->dq_strides[2];
  p.dk_bs = a->dk_strides[0]; p.dk_rs = a->dk_strides[1]; p.dk_hs = a->dk_strides[2];
  p.dv_bs = a->dv_strides[0]; p.dv_rs = a->dv_strides[1]; p.dv_hs = a->dv_strides[2];
  p.seq_q = a->seq_q; p.seq_k = a->seq_k; p.heads = a->heads; p.kv_heads = a->kv_heads; p.causal = a->causal;
  p.scale = a->scale;
  return true;
}
bool strides_ok(const long long* s) { return (s[0] % 8 == 0) && (s[1] % 8 == 0) && (s[2] % 8 == 0); }
bool ptr_ok(const void* p) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
}  // namespace

RB_API int rb_attention_fwd(const RbAttnArgs* a, void* stream_v) {
  if (a->kv_lens) return -9;                 // key-padding lengths are not implemented by the mma.sync kernels
  rb::AttnParams p;
  if (!fill_params(a, p)) return -1;
  if (!ptr_ok(a->q) || !ptr_ok(a->k) || !ptr_ok(a->v) || !ptr_ok(a->o)) return -2;
  if (!strides_ok(a->q_strides) || !strides_ok(a->k_strides) || !strides_ok(a->v_strides) || !strides_ok(a->o_strides)) return -2;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  dim3 grid((a->seq_q + rb::kTile - 1) / rb::kTile, a->heads, a->batch);
  const int smem = 5 * rb::kTile * a->head_dim * 2;
  if (a->head_dim == 64) {
    rb::attn_fwd_kernel<64><<<grid, rb::kAttnThreads, smem, stream>>>(p);
  } else {
    static bool cfg_dev[64] = {false};
    bool& cfg = cfg_dev[rbhost::device_slot()];
    if (!cfg) { cudaFuncSetAttribute(rb::attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); cfg = true; }
    rb::attn_fwd_kernel<128><<<grid, rb::kAttnThreads, smem, stream>>>(p);
  }
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_attention_bwd(const RbAttnArgs* a, void* stream_v) {
  if (a->kv_lens) return -9;                 // key-padding lengths are not implemented by the mma.sync kernels
  rb::AttnParams p;
  if (!fill_params(a, p)) return -1;
  if (!ptr_ok(a->q) || !ptr_ok(a->k) || !ptr_ok(a->v) || !ptr_ok(a->o) || !ptr_ok(a->d_o) || !ptr_ok(a->dq) ||
      !ptr_ok(a->dk) || !ptr_ok(a->dv) || !a->lse || !a->delta)
    return -2;
  if (!strides_ok(a->q_strides) || !strides_ok(a->k_strides) || !strides_ok(a->v_strides) || !strides_ok(a->o_strides) ||
      !strides_ok(a->dq_strides) || !strides_ok(a->dk_strides) || !strides_ok(a->dv_strides))
    return -2;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const long long rows = static_cast<long long>(a->heads) * a->seq_q;
  dim3 dgrid(static_cast<unsigned>((rows + 3) / 4), a->batch);
  dim3 kvgrid((a->seq_k + rb::kTile - 1) / rb::kTile, a->kv_heads, a->batch);
  dim3 qgrid((a->seq_q + rb::kTile - 1) / rb::kTile, a->heads, a->batch);
  const int smem_kv = 6 * rb::kTile * a->head_dim * 2 + 4 * rb::kTile * static_cast<int>(sizeof(float));
  const int smem_q = 6 * rb::kTile * a->head_dim * 2;
  if (a->head_dim == 64) {
    static bool cfg_dev[64] = {false};
    bool& cfg = cfg_dev[rbhost::device_slot()];
    if (!cfg) {
      cudaFuncSetAttribute(rb::attn_bwd_dkv_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_kv);
      cudaFuncSetAttribute(rb::attn_bwd_dq_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_q);
      cfg = true;
    }
    rb::attn_delta_kernel<64><<<dgrid, 128, 0, stream>>>(p);
    rb::attn_bwd_dkv_kernel<64><<<kvgrid, rb::kAttnThreads, smem_kv, stream>>>(p);
    rb::attn_bwd_dq_kernel<64><<<qgrid, rb::kAttnThreads, smem_q, stream>>>(p);
  } else {
    static bool cfg_dev[64] = {false};
    bool& cfg = cfg_dev[rbhost::device_slot()];
    if (!cfg) {
      cudaFuncSetAttribute(rb::attn_bwd_dkv_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_kv);
      cudaFuncSetAttribute(rb::attn_bwd_dq_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_q);
      cfg = true;
    }
    rb::attn_delta_kernel<128><<<dgrid, 128, 0, stream>>>(p);
    rb::attn_bwd_dkv_kernel<128><<<kvgrid, rb::kAttnThreads, smem_kv, stream>>>(p);
    rb::attn_bwd_dq_kernel<128><<<qgrid, rb::kAttnThreads, smem_q, stream>>>(p);
  }
  return static_cast<int>(cudaGetLastError());
}
