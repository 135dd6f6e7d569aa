// C interface of the softmax / cross-entropy kernels (loss.cu).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// Fused softmax-cross-entropy forward + backward over bf16 logits [rows, n_valid] with pitch ld.
//   loss[r]   = logsumexp(logits[r, :n_valid]) - logits[r, target[r]]      (0 where target == ignore_index)
//   dlogits   = (softmax - onehot) * grad_scale, written in bf16 (may alias logits); columns
//               [n_valid, n_pad) are written as zero so a padded vocabulary stays inert.
// dlogits may be NULL (forward only).  lse (fp32 [rows]) may be NULL.
int rb_cross_entropy(const void* logits, long long ld, const long long* targets, float* loss, float* lse,
                     void* dlogits, long long ldd, int rows, int n_valid, int n_pad, float grad_scale,
                     long long ignore_index, void* stream);
// Vocabulary-parallel tail of the cross-entropy: this rank holds columns of the logits, `lse` is the log-sum-exp over
// ALL ranks' columns.  dlogits[r, c] = (exp(logits[r, c] - lse[r]) - [c == targets[r]]) * grad_scale, bf16, may alias
// logits.  targets are LOCAL column indices; rows whose target lives on another rank carry a value outside [0, n).
int rb_cross_entropy_grad_lse(const void* logits, long long ld, const long long* targets, const float* lse, void* dlogits,
                              long long ldd, int rows, int n, float grad_scale, void* stream);
// Row softmax / log-softmax over the last dimension, fp32 or bf16 in and out (dtype: 0 = fp32, 1 = bf16).
int rb_softmax_rows(const void* x, void* y, int rows, int n, long long ldx, long long ldy, int log_mode, int dtype,
                    void* stream);
// y[r, :] = grad of softmax (log_mode 0) or log-softmax (log_mode 1) given the forward OUTPUT `out` and upstream `dy`; fp32.
int rb_softmax_rows_bwd(const float* out, const float* dy, float* dx, int rows, int n, int log_mode, void* stream);
#ifdef __cplusplus
}
#endif
