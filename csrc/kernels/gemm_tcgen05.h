// C interface of the tcgen05 bf16 GEMM (see gemm_tcgen05.cu).  Plain C so that it can be bound
// with ctypes; every pointer is a device pointer.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

enum RbAct {
  RB_ACT_NONE = 0,
  RB_ACT_GELU = 1,    // tanh-approximated GELU (the reference's definition, crates/ndarray-backend/src/lib.rs:565)
  RB_ACT_RELU = 2,
  RB_ACT_SILU = 3,
  RB_ACT_DGELU = 4,   // multiply the result by gelu'(aux_in)
  RB_ACT_DRELU = 5,   // zero the result where aux_in <= 0
  RB_ACT_DSILU = 6,   // multiply the result by silu'(aux_in)
  RB_ACT_MUL = 7      // multiply the result by aux_in
};

typedef struct RbGemmArgs {
  const void* a;        // bf16; K-major: [M,K] pitch lda; MN-major: [K,M] pitch lda
  const void* b;        // bf16; K-major: [N,K] pitch ldb; MN-major: [K,N] pitch ldb
  void* d;              // [M,N] pitch ldd, bf16 or fp32
  const void* bias;     // bf16 [N] or NULL, added before the activation
  const void* residual; // bf16 [M,N] pitch ldr or NULL, added after the activation
  const void* aux_in;   // bf16 [M,N] pitch ld_aux_in, operand of the RB_ACT_D* / RB_ACT_MUL epilogues
  void* aux_out;        // bf16 [M,N] pitch ld_aux_out or NULL: receives the pre-activation
  long long lda, ldb, ldd, ldr, ld_aux_in, ld_aux_out;
  int M, N, K;
  int a_mn_major, b_mn_major;
  int act;              // RbAct
  int out_f32;          // 1: d is fp32
  int accumulate;       // 1: d += result
  float alpha;          // scales the accumulator before everything else
  int block_n;          // 0 = choose; else 64 / 128 / 192 / 256
  int group_m;          // 0 = default (8): M-tiles per rasterisation group
  int max_ctas;         // 0 = one per SM; else cap on the persistent grid
  int splits;           // 0 = choose (split-K only when a workspace is given); 1 = never split; else forced count
  void* workspace;      // fp32 scratch for split-K partial sums (splits * M * N floats), or NULL
  long long workspace_bytes;
  // grouped (mixture-of-experts) execution; all pointers are device int32 arrays
  int group_mode;       // 0 off; 1 rows of A/D grouped by expert, B stacked per expert; 2 one D per expert, K ranges per expert
  int num_experts;
  const void* tile_expert;     // mode 1: expert of every 128-row tile of A (-1 = none)
  const void* num_m_tiles;     // mode 1: [1] number of live 128-row tiles
  const void* expert_offsets;  // mode 2: [num_experts + 1] row offsets (multiples of 128) into A and B
  int b_expert_rows;           // mode 1: rows of B per expert (N for K-major B, K for MN-major B)
  long long d_expert_stride;   // mode 2: elements between consecutive experts' outputs
  // fusion with tensor-parallel collectives over peer memory (NVLink); see PeerInfo in gemm_tcgen05.cu
  int peer_mode;               // 0 off; 1 all-gather(A rows) -> GEMM; 2 GEMM -> reduce-scatter (stores into the owners'
                               // slots); 3 all-gather(B rows, a row-sharded weight) -> GEMM
  int peer_world, peer_rank;
  int rows_per_rank;           // M / peer_world (mode 3: N / peer_world), a multiple of 128
  unsigned int peer_epoch;     // mode 1 / 3: call counter of this workspace (the block counters reach 32 * epoch)
  void* ready_flags;           // mode 1 / 3: local u32 counters, one per 128-row block of the gathered operand
  const void* peer_ptrs[8];    // mode 1 / 3: every rank's shard [rows_per_rank, K] of A / B; mode 2: every rank's receive buffer
                               //         [peer_world][rows_per_rank, ldd] (this rank writes slot peer_rank)
  // 8-bit floating-point operands (tcgen05 kind::f8f6f4, fp32 accumulation): a and b hold e4m3 bytes, both K-major,
  // lda / ldb / K count bytes (multiples of 16).  Plain and grouped mode 1 problems only.  For every operand type the
  // accumulator of row i, column j is multiplied by a_scale[i] * b_scale[j] (each may be NULL) before the bias.
  // grouped mode 1 fed by an expert-parallel dispatch that is still in flight: tile_arrived[i] (device u32, written by
  // the ranks that store rows of 128-row tile i of A) is waited for (bounded) to reach tile_expected[i] before tile i
  // of A is loaded.  Both NULL: A is complete when the kernel starts.
  const void* tile_arrived;
  const void* tile_expected;
  int ab_fp8;                  // 0: bf16 operands; 1: a and b e4m3; 2: a e4m3, b e5m2
  const void* a_scale;         // fp32 [M] or NULL: one scale per row of A (per token)
  const void* b_scale;         // fp32 [N] or NULL: one scale per row of B (per output channel)
} RbGemmArgs;

// Returns 0 on success, a negative code for rejected arguments, a positive cudaError otherwise.
int rb_gemm_bf16(const RbGemmArgs* args, void* stream);

#ifdef __cplusplus
}
#endif
