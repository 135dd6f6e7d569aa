// C interface of the optimizer kernels (optim.cu).  All state is fp32 and flat; parameters are
// kept twice: an fp32 master copy that the optimizer updates and a bf16 working copy for the GEMMs.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
typedef struct RbAdamArgs {
  float lr, beta1, beta2, eps, weight_decay;
  float bias_correction1, bias_correction2;   // 1 - beta^t, computed by the caller
  float grad_scale;                           // multiplies the gradient first (1 / loss scale / accumulation)
  int decoupled;                              // 1: AdamW (p -= lr*wd*p), 0: L2 folded into the gradient
  float max_grad_norm;                        // <= 0: no clipping; else clip by *grad_norm (a device scalar)
} RbAdamArgs;

// p, m, v: fp32 [n]; g: fp32 [n] or bf16 [n] (g_bf16 = 1); p_bf16: optional bf16 [n] working copy.
// grad_norm: optional device float holding the global L2 norm of grad_scale * g (for clipping).
// found_inf: optional device int; when non-zero on entry the step is skipped on the device.
int rb_adam_step(float* p, float* m, float* v, const void* g, int g_bf16, void* p_bf16, long long n,
                 const RbAdamArgs* args, const float* grad_norm, const int* found_inf, void* stream);
int rb_sgd_step(float* p, float* mom, const void* g, int g_bf16, void* p_bf16, long long n, float lr, float momentum,
                float weight_decay, float grad_scale, void* stream);
// out[0] += sum(x^2) (fp32 accumulate; clear out first), found_inf set to 1 when a non-finite value is seen.
// Two-stage and ordered, so the result is reproducible.  scratch: >= rb_sumsq_scratch_floats() floats.
int rb_sumsq_scratch_floats(void);
int rb_sumsq(const void* x, int is_bf16, long long n, float* scratch, float* out, int* found_inf, int accumulate,
             void* stream);
// out[0] = sqrt(in[0])
int rb_sqrt_scalar(const float* in, float* out, void* stream);
// dst (bf16) = src (fp32) and the reverse
int rb_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream);
int rb_cast_bf16_to_f32(const void* src, float* dst, long long n, void* stream);
#ifdef __cplusplus
}
#endif
