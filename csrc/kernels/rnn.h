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
#ifdef __cplusplus
}
#endif
