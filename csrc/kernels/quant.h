// C interface of the quantisation kernels (quant.cu).  All pointers are device pointers.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// bf16 [rows, n] (pitch ldx elements) -> e4m3 bytes [rows, n] (pitch ldo bytes) and scales[row] = absmax / 448 (1 for an
// all-zero row), so that x ~= scale * e4m3.  n, ldo multiples of 16; ldx a multiple of 8.
int rb_quantize_fp8_rows(const void* x, long long ldx, void* out, long long ldo, void* scales, int rows, int n, void* stream);
// int8 [rows, n] dense -> bf16 (q - zero_point), exact.  zero_point: fp32 [rows] (zp_per_row = 1), [1] (0) or NULL.
int rb_dequant_int8_bf16(const void* q, const void* zero_point, int zp_per_row, void* out, int rows, int n, void* stream);
// nibbles [rows, n / 2] (element 2b in the low half of byte b) with scales fp32 [rows, n / group_size] -> bf16
// (q - 8) * scale.  n and group_size multiples of 32.
int rb_dequant_int4_bf16(const void* packed, const void* scales, int group_size, void* out, int rows, int n, void* stream);
#ifdef __cplusplus
}
#endif
