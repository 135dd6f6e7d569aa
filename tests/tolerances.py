"""Per-element tolerances of the GPU numerics tests, one entry per family of kernels.

A check passes when, for every element, |out - ref| <= atol_frac * max|ref| + rtol * |ref|: the relative term bounds
the rounding of the output format, the absolute term (a fraction of the largest reference magnitude) covers what
cancellation leaves of the accumulation error in elements close to zero.

    family               output   why these numbers
    gemm_f32             fp32     bf16 inputs are exact in fp32; what differs is the fp32 accumulation order
    gemm_bf16            bf16     one rounding to bf16 (2^-9 relative) on top of the fp32 accumulation
    gemm_act             bf16     + tanh.approx (2^-11) in the GELU epilogue
    attention            bf16     P rounded to bf16 before PV, ex2.approx, output rounded to bf16
    attention_grad       bf16     two more bf16-rounded operands (dS, P) per product
    norm                 bf16     fp32 statistics, bf16 output
    reduce_f32           fp32     ordered fp32 sums against torch's pairwise sums
"""
import torch

TABLE = {
    "gemm_f32": (2e-5, 1e-4),
    "gemm_bf16": (1e-3, 5e-3),
    "gemm_act": (2e-3, 8e-3),
    "attention": (4e-3, 1e-2),
    "attention_grad": (8e-3, 2e-2),
    "norm": (2e-3, 8e-3),
    "reduce_f32": (1e-5, 1e-4),
}


def assert_close(out: torch.Tensor, ref: torch.Tensor, family: str, what: str = "") -> None:
    atol_frac, rtol = TABLE[family]
    out, ref = out.detach().float().cpu(), ref.detach().float().cpu()
    assert out.shape == ref.shape, f"{what}: shape {tuple(out.shape)} != {tuple(ref.shape)}"
    bound = atol_frac * ref.abs().max() + rtol * ref.abs()
    excess = (out - ref).abs() - bound
    worst = int(excess.argmax())
    assert excess.flatten()[worst] <= 0, (
        f"{what or family}: element {worst}: out {out.flatten()[worst].item():.6g} ref {ref.flatten()[worst].item():.6g} "
        f"bound {bound.flatten()[worst].item():.3g} ({family}: atol {atol_frac:g} x max|ref|, rtol {rtol:g})")
