// C interface of the elementwise / reduction / data-movement kernel family (elementwise.cu).
// dtype: 0 = fp32, 1 = bf16.  All pointers are device pointers.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
enum RbBinaryOp { RB_ADD = 0, RB_MUL = 1, RB_SUB = 2, RB_DIV = 3, RB_MAXIMUM = 4 };
enum RbUnaryOp {
  RB_RELU = 0, RB_SIGMOID = 1, RB_TANH = 2, RB_EXP = 3, RB_LOG = 4, RB_SQRT = 5, RB_NEG = 6, RB_GELU = 7,
  RB_SILU = 8, RB_COPY = 9
};
enum RbScalarOp { RB_ADD_SCALAR = 0, RB_MUL_SCALAR = 1, RB_GT_SCALAR = 2, RB_FILL = 3 };

int rb_binary(int op, const void* a, const void* b, void* out, long long n, int dtype, void* stream);
int rb_unary(int op, const void* a, void* out, long long n, int dtype, void* stream);
int rb_scalar(int op, const void* a, float s, void* out, long long n, int dtype, void* stream);
// out = dy * act'(x) for RB_RELU / RB_GELU / RB_SILU / RB_SIGMOID / RB_TANH
int rb_unary_bwd(int op, const void* x, const void* dy, void* out, long long n, int dtype, void* stream);
// out[r, c] = a[r, c] + v[c]
int rb_add_row_vector(const void* a, const void* v, void* out, long long rows, int cols, int dtype, void* stream);
// out[c] (+)= sum_r a[r, c]; input fp32 or bf16, output fp32; ordered, reproducible
int rb_sum_dim0(const void* a, long long lda, float* out, long long rows, int cols, int dtype, int accumulate, void* stream);
// Same sum in two ordered stages spread over many CTAs; partial holds rb_sum_dim0_slabs() * cols floats.
int rb_sum_dim0_slabs(void);
int rb_sum_dim0_staged(const void* a, long long lda, float* out, float* partial, long long rows, int cols, int dtype,
                       int accumulate, void* stream);
// out[0] = sum(a); scratch >= 1024 floats
int rb_sum_all(const void* a, long long n, int dtype, float* scratch, float* out, void* stream);
// 2-D transpose out[c, r] = a[r, c]
int rb_transpose(const void* a, void* out, int rows, int cols, int dtype, void* stream);
// out[i, :] = a[idx[i], :]; scatter: out[idx[i], :] = a[i, :] (last writer wins, as in the reference's scatter_rows)
int rb_gather_rows(const void* a, const long long* idx, void* out, long long n_idx, int cols, long long src_rows, int dtype, void* stream);
int rb_scatter_rows(const void* a, const long long* idx, void* out, long long n_idx, int cols, long long dst_rows, int dtype, void* stream);
// out[r, c] = a[r % arows, c % acols]
int rb_broadcast_to(const void* a, void* out, long long arows, long long acols, long long rows, long long cols, int dtype, void* stream);
// 2-D strided copy: out[r*ldo + c] = a[r*lda + c]
int rb_strided_copy(const void* a, long long lda, void* out, long long ldo, long long rows, long long cols, int dtype, void* stream);
// out = mask > 0 ? a : mask_value   (mask has the dtype of a)
int rb_apply_mask(const void* a, const void* mask, float mask_value, void* out, long long n, int dtype, void* stream);
// Inverted dropout.  rng 0: Philox-4x32-10 keyed by (seed, offset); rng 1: the PCG hash of `seed + idx*12345`
// (the generator of the reference's WGSL dropout, shaders.wgsl:1238-1281).  mask_out (uint8, optional) gets the keep mask.
int rb_dropout(const void* a, void* out, unsigned char* mask_out, long long n, float p, unsigned long long seed,
               unsigned long long offset, int rng, int dtype, void* stream);
// out[r] = argmax_c a[r, c]
int rb_argmax_rows(const void* a, long long lda, long long* out, long long rows, int cols, int dtype, void* stream);
#ifdef __cplusplus
}
#endif
