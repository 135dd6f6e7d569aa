// C interface of the direct convolution kernel (conv.cu).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// y[n, o, ho, wo] = bias[o] + sum over c, i, j of x[n, c, ho * stride - pad_h + i, wo * stride - pad_w + j] * w[o, c, i, j]
// x [N, C, H, W], w [O, C, kh, kw], bias [O] or NULL, y [N, O, Ho, Wo] with Ho = (H + 2 pad_h - kh) / stride + 1
// (Wo likewise); all bf16 and dense, fp32 accumulation, taps outside the image read zero.  The filter bank is held in
// shared memory as fp32: O * C * kh * kw may not exceed 12288 (48 KB), larger banks are refused with -3 and belong
// on the im2col + GEMM path.
int rb_conv2d_fwd(const void* x, const void* w, const void* bias, void* y, int N, int C, int H, int W, int O, int kh, int kw,
                  int stride, int pad_h, int pad_w, void* stream);
#ifdef __cplusplus
}
#endif
