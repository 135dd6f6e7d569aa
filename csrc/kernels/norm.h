// C interface of the LayerNorm / RMSNorm kernels (norm.cu).  All pointers are device pointers;
// activations and parameters are bf16, statistics and parameter gradients fp32.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// Number of partial rows the backward pass writes for a [rows, n] problem; the scratch buffer handed
// to rb_norm_bwd must hold 2 * that * n floats.
int rb_norm_bwd_num_partials(int rows, int n);
int rb_norm_fwd(const void* x, long long ldx, const void* gamma, const void* beta, void* y, long long ldy,
                float* mean, float* rstd, int rows, int n, float eps, int rms, void* stream);
int rb_norm_bwd(const void* dy, long long lddy, const void* x, long long ldx, const void* gamma, const float* mean,
                const float* rstd, const void* dres, long long lddres, void* dx, long long lddx, float* dgamma,
                float* dbeta, float* partial, int rows, int n, int rms, int accumulate, void* stream);
#ifdef __cplusplus
}
#endif
