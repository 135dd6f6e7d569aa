// C interface of the recurrent-cell kernels (rnn.cu).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// LSTM cell update from pre-activations.  gates [B, 4H] bf16 with row pitch ld_g, gate order i | f | o | g (the sum
// x W_x^T + h W_h^T + b); c_prev, h_out, c_out [B, H] bf16, dense.  In fp32:
//   c = sigmoid(f) * c_prev + sigmoid(i) * tanh(g);   h = sigmoid(o) * tanh(c)
// h_out / c_out may alias c_prev.  H must be even.
int rb_lstm_gates_fwd(const void* gates, long long ld_g, const void* c_prev, void* h_out, void* c_out, int B, int H,
                      void* stream);
// Backward of the update above: dgates [B, 4H] (pitch ld_dg) and dc_prev [B, H] from dh, dc_out (NULL = zero), the saved
// pre-activations, c_prev and c_out.
int rb_lstm_gates_bwd(const void* gates, long long ld_g, const void* c_prev, const void* c_out, const void* dh, const void* dc_out,
                      void* dgates, long long ld_dg, void* dc_prev, int B, int H, void* stream);
// GRU cell update from the two projections gx = x W_x^T + b and gh = h W_h^T, [B, 3H] each in the order r | z | n:
//   r = sigmoid(gx_r + gh_r); z = sigmoid(gx_z + gh_z); n = tanh(gx_n + r * gh_n); h = (1 - z) * n + z * h_prev
int rb_gru_gates_fwd(const void* gx, long long ld_x, const void* gh, long long ld_h, const void* h_prev, void* h_out, int B, int H,
                     void* stream);
// Its backward: dgx, dgh (dense [B, 3H]) and dh_prev from dh.
int rb_gru_gates_bwd(const void* gx, long long ld_x, const void* gh, long long ld_h, const void* h_prev, const void* dh, void* dgx,
                     void* dgh, void* dh_prev, int B, int H, void* stream);
#ifdef __cplusplus
}
#endif
