// C interface of the expert-choice routing kernels (expert_choice.cu).  All pointers are device pointers.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// probs [T, E] fp32.  For every expert e: idx[e * cap + s] (int64) = its s-th chosen token, ascending token order, and
// gate[e * cap + s] = probs[token, e].  Chosen are the cap largest probabilities of column e; ties at the threshold go to
// the lower token index.  cap <= T.
int rb_ec_select(const float* probs, int T, int E, int cap, long long* idx, float* gate, void* stream);
// table [T, E] int32: position of token t in expert e's list, -1 when e did not choose t.
int rb_ec_table(const long long* idx, int T, int E, int cap, int* table, void* stream);
// out[t, :] = sum over e ascending of gate[e * cap + s] * y[e * cap + s, :], s = table[t, e] >= 0; tokens nobody chose get
// zeros.  y [E * cap, d] bf16; gate fp32 or NULL (unit weights); out bf16 or fp32 (out_f32); d a multiple of 8.
int rb_ec_combine(const void* y, const float* gate, const int* table, void* out, int T, int E, int cap, int d, int out_f32, void* stream);
// dy[j, :] = gate[j] * dout[idx[j], :] (bf16) and, when y and dgate are given, dgate[j] = <dout[idx[j], :], y[j, :]>.
int rb_ec_combine_bwd(const void* dout, const long long* idx, const float* gate, const void* y, void* dy, float* dgate, int n, int T,
                      int d, void* stream);
#ifdef __cplusplus
}
#endif
