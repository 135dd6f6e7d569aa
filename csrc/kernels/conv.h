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
// Convolution as a GEMM over unfolded patches (training, large filter banks); all tensors bf16 and dense.
//   rb_im2col: x [N, C, H, W] -> cols [N * Ho * Wo, Kp], column (c, i, j) of row (n, ho, wo) holds the tap's pixel (zero
//   outside the image); columns from C * kh * kw up to Kp are zero.   rb_col2im: its adjoint, dcols -> dx, no atomics.
int rb_im2col(const void* x, void* cols, int N, int C, int H, int W, int kh, int kw, int stride, int pad_h, int pad_w, int Kp, void* stream);
int rb_col2im(const void* dcols, void* dx, int N, int C, int H, int W, int kh, int kw, int stride, int pad_h, int pad_w, int Kp, void* stream);
//   rb_nhwc_to_nchw: src [N * L, ld_src] (first O columns) -> dst [N, O, L];  rb_nchw_to_nhwc: src [N, O, L] -> dst [N * L, Op]
//   with zeros in columns [O, Op).
int rb_nhwc_to_nchw(const void* src, long long ld_src, void* dst, int N, int L, int O, void* stream);
int rb_nchw_to_nhwc(const void* src, void* dst, int N, int L, int O, int Op, void* stream);
// Max pooling without padding over `planes` = N * C images of H x W (dense): y [planes, Ho, Wo], idx (int32) the flat
// position h * W + w of each window's maximum; Ho = (H - k) / stride + 1.  Backward: dx[p] = sum of dy over the windows
// whose maximum is p (a gather, no atomics).  bf16 or fp32 elements.
int rb_max_pool2d_fwd(const void* x, void* y, int* idx, long long planes, int H, int W, int k, int stride, int is_bf16, void* stream);
int rb_max_pool2d_bwd(const void* dy, const int* idx, void* dx, long long planes, int H, int W, int k, int stride, int is_bf16, void* stream);
#ifdef __cplusplus
}
#endif
