// C interface of the expert-parallel dispatch / combine kernels (ep.cu).  Tokens move between GPUs with plain peer
// stores (dispatch: straight into the destination rank's grouped-GEMM operand buffer) and peer loads (combine:
// straight out of the expert ranks' output buffers); the caller orders them with the signal-pad flags of symm.h.
// Per (token, choice) pair p the maps give the destination rank and the row inside that rank's buffer.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// dst[dest_rank[p]][dest_row[p], :] = src[p / k, :] * (scale ? scale[p] : 1)      (bf16 rows of d elements, d % 8 == 0)
// peer_counts_dev (optional): per rank a u32 array with one counter per 128-row tile of its buffer; every stored row
// adds one to its tile's counter on the owner (system-scope release), which the owner's grouped GEMM waits on per tile.
int rb_ep_push_rows(const void* src, int tokens, int k, int d, const int* dest_rank, const int* dest_row,
                    const float* scale, void* const* peer_bufs_dev, void* const* peer_counts_dev, void* stream);
// out[t, :] = sum_j (w ? w[t*k+j] : 1) * buf[dest_rank[p]][dest_row[p], :] (+ residual[t, :]),  p = t*k + j, j ascending
int rb_ep_pull_combine(void* out, int tokens, int k, int d, const int* dest_rank, const int* dest_row, const float* w,
                       const void* residual, void* const* peer_bufs_dev, void* stream);
// dw[t*k+j] = < dy[t, :], buf[dest_rank[p]][dest_row[p], :] >
int rb_ep_pull_dot(float* dw, const void* dy, int tokens, int k, int d, const int* dest_rank, const int* dest_row,
                   void* const* peer_bufs_dev, void* stream);
// Zero the padding rows [offsets[e] + counts[e], offsets[e+1]) of every local expert segment of a receive buffer.
int rb_ep_zero_padding(void* buf, const int* offsets, const int* counts, int num_local_experts, int d, void* stream);
#ifdef __cplusplus
}
#endif
