// C interface of the C++ f32 reference backend (librb200_cpu.so): the numerical oracle for every CUDA kernel and
// the timed CPU baseline.  Row-major f32 everywhere.  Mirrors the op table of the reference's CPU backend
// (crates/ndarray-backend/src/lib.rs:169-1746) with the intended semantics where that file deviates.
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
void rb_cpu_set_threads(int n);                       // 0 = hardware concurrency
// c[m,n] = a[m,k] * b[k,n]
void rb_cpu_matmul(const float* a, const float* b, float* c, int m, int k, int n);
// y[batch,out] = act(x[batch,in] * w[out,in]^T + bias);  act: 0 none, 1 gelu(tanh), 2 relu, 3 silu
void rb_cpu_linear(const float* x, const float* w, const float* bias, float* y, int batch, int in, int out, int act);
void rb_cpu_softmax_rows(const float* x, float* y, int rows, int n, int log_mode);
// population variance, eps inside the square root; gamma/beta may be NULL; rms = 1 selects RMSNorm
void rb_cpu_layer_norm(const float* x, const float* gamma, const float* beta, float* y, float* mean, float* rstd,
                       int rows, int n, float eps, int rms);
void rb_cpu_layer_norm_bwd(const float* dy, const float* x, const float* gamma, const float* mean, const float* rstd,
                           float* dx, float* dgamma, float* dbeta, int rows, int n, int rms);
void rb_cpu_unary(int op, const float* x, float* y, int64_t n);          // op codes of elementwise.h (RbUnaryOp)
// loss[r] = logsumexp(logits[r,:]) - logits[r,target[r]]; dlogits = (softmax - onehot) * scale (may be NULL)
void rb_cpu_cross_entropy(const float* logits, const int64_t* targets, float* loss, float* dlogits, int rows, int n,
                          float scale, int64_t ignore_index);
void rb_cpu_adam(float* p, float* m, float* v, const float* g, int64_t n, float lr, float b1, float b2, float eps,
                 float wd, int step, int decoupled);
// q [B,S,H,D], k/v [B,Sk,Hkv,D] -> o [B,S,H,D]; causal aligns queries to the end of the keys
void rb_cpu_attention(const float* q, const float* k, const float* v, float* o, int B, int Sq, int Sk, int H, int Hkv,
                      int D, int causal, float scale);
// router: probs = softmax(logits[T,E]); top-k per token (descending, ties to the lower index); weights renormalised
// when renorm != 0.  aux = E * sum_e f_e * P_e (fraction routed x mean probability).
void rb_cpu_moe_route(const float* logits, int T, int E, int k, int renorm, int32_t* idx_out, float* w_out, float* aux_out);
void rb_cpu_gather_rows(const float* table, const int64_t* ids, float* out, int64_t n_ids, int cols, int64_t rows);
void rb_cpu_scatter_add_rows(const float* src, const int64_t* ids, float* table, int64_t n_ids, int cols, int64_t rows);
#ifdef __cplusplus
}
#endif
