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

// ---- allocation-free variant (an addition of this library; the reference has nothing like it) ----------------------
// Same computation and the same arguments as rb_norm_bwd minus the scratch pointer: the partial sums live in a
// fixed device array inside the library instead of in memory the caller allocated.  It is meant for callers that
// may not allocate device memory where they run: code inside a region where cudaMalloc is forbidden or would
// synchronise the device (an inference server's steady state, a real-time loop, a plugin handed only its input and
// output buffers), or host code that has no allocator to borrow from.  The entry point itself calls no cudaMalloc,
// cudaFree or any allocating library routine.
//
// Limits and rules:
//   * 2 * rb_norm_bwd_num_partials(rows, n) * n must not exceed rb_norm_bwd_noalloc_capacity_floats()
//     (2 * 296 * 4096 floats, 9.25 MiB); larger problems are refused with -22 and nothing is launched.
//     Every row length the kernels support up to 4096 fits for any number of rows.
//   * The first call on a device looks up the device address of the built-in array (cudaGetSymbolAddress, with that
//     device current) and remembers it; make that first call outside any stream capture.
//   * All calls on one device share the one array.  Calls whose kernels may overlap on the GPU (different streams
//     without an ordering between them) race on it; keep them on one stream or order them with events.
//   * Return codes: 0 success; -20 / -21 the device or the array's address could not be determined; -22 too large;
//     otherwise the codes of rb_norm_bwd.
long long rb_norm_bwd_noalloc_capacity_floats(void);
int rb_norm_bwd_noalloc(const void* dy, long long lddy, const void* x, long long ldx, const void* gamma, const float* mean,
                        const float* rstd, const void* dres, long long lddres, void* dx, long long lddx, float* dgamma,
                        float* dbeta, int rows, int n, int rms, int accumulate, void* stream);
#ifdef __cplusplus
}
#endif
