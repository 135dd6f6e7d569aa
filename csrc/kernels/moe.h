// C interface of the mixture-of-experts routing / permutation kernels (moe.cu).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
#define RB_MOE_ROW_ALIGN 128   // every expert's segment of the permuted buffer starts on a multiple of this many rows

// Router: probs = softmax(logits[T, E]) per token (fp32), top-k experts per token (descending probability, ties to
// the lower index).  idx [T, k] int32, w [T, k] fp32 (renormalised over the selected experts when renorm != 0),
// probs_out [T, E] fp32 (optional, needed by the backward pass).  E <= 64, k <= 8.
int rb_moe_route(const float* logits, int T, int E, int k, int renorm, int* idx, float* w, float* probs_out, void* stream);
// Backward of the router: dlogits [T, E] fp32 from dw [T, k] and the load-balancing loss
//   aux = E * sum_e f_e * P_e,  f_e = (tokens routed to e) / (T k),  P_e = mean_t probs[t, e]
// aux_grad_scale multiplies d aux (pass coefficient * upstream gradient).  counts: int32 [E] tokens per expert.
int rb_moe_route_bwd(const float* probs, const int* idx, const float* w, const float* dw, const int* counts, int T, int E,
                     int k, int renorm, float aux_grad_scale, float* dlogits, void* stream);
// Plan of the permutation: slots s = t * k + j are grouped by expert, in ascending slot order inside an expert
// (deterministic).  Outputs (all device memory):
//   counts [E]            tokens per expert
//   offsets [E + 1]       first row of each expert in the permuted buffer, multiples of RB_MOE_ROW_ALIGN
//   slot_pos [T * k]      row of every slot in the permuted buffer
//   row_slot [max_rows]   slot of every row, -1 for padding rows; max_rows >= T * k + E * RB_MOE_ROW_ALIGN
//   tile_expert [max_rows / 128]  expert of every 128-row tile, -1 past the end;  num_tiles [1]
int rb_moe_plan(const int* idx, int T, int E, int k, int* counts, int* offsets, int* slot_pos, int* row_slot,
                int* tile_expert, int* num_tiles, int max_rows, void* stream);
// xp[r, :] = scale(r) * x[row_slot[r] / k, :], zero for padding rows.  row_scale (fp32 [T * k], optional) is indexed by slot.
int rb_moe_gather(const void* x, const int* row_slot, const float* slot_scale, void* xp, int max_rows, int k, int dim,
                  const int* offsets_last, void* stream);
// y[t, :] = sum_j w[t, j] * yp[slot_pos[t * k + j], :] (+ residual[t, :]); w == NULL means unit weights.
int rb_moe_combine(const void* yp, const int* slot_pos, const float* w, const void* residual, void* y, int T, int k, int dim,
                   void* stream);
// dw[s] = <dy[s / k, :], yp[slot_pos[s], :]>
int rb_moe_weight_grad(const void* dy, const void* yp, const int* slot_pos, float* dw, int T, int k, int dim, void* stream);
#ifdef __cplusplus
}
#endif
