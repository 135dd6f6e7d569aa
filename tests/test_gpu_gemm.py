"""tcgen05 GEMM against an fp32 reference of the same product (bf16 inputs rounded identically)."""
import pytest
import torch

from rustral_b200 import ops
from rustral_b200.ops.matmul import act_reference, act_grad_reference

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    return A @ B.t()


def _mk(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * 0.5).to(torch.bfloat16)


from tolerances import assert_close


def _close(out, ref, tol=None, family=None):
    """Per-element check against the table in tests/tolerances.py: fp32 outputs of fp32-accumulated products are held
    to 1e-4 relative, bf16 outputs to their rounding, epilogues with an activation to the approximation they use."""
    if family is None:
        family = "gemm_f32" if out.dtype == torch.float32 else ("gemm_act" if (tol or 0) > 2e-2 else "gemm_bf16")
    assert_close(out, ref, family)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 128), (256, 128, 256), (130, 72, 96), (1000, 768, 776),
                                   (64, 64, 64), (8, 8, 8), (2048, 2304, 768)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_majors(M, N, K, a_mn, b_mn, cuda_status):
    # a transposed operand's row pitch is M (or N) elements and TMA needs 16-byte pitches: (130, ...) with a_mn runs on
    # zero-padded copies (ops.matmul._gemm_padded) and must give the same result as every other case
    a = _mk((K, M) if a_mn else (M, K), 1)
    b = _mk((K, N) if b_mn else (N, K), 2)
    ref = _ref(a, b, a_mn, b_mn)
    out = ops.gemm(a.cuda(), b.cuda(), a_mn=a_mn, b_mn=b_mn)
    assert out.dtype == torch.bfloat16 and out.shape == (M, N)
    _close(out, ref)


@pytest.mark.parametrize("block_n", [64, 128, 192, 256])
def test_gemm_block_n(block_n, cuda_status):
    M, N, K = 384, 512, 320
    a, b = _mk((M, K), 3), _mk((N, K), 4)
    out = ops.gemm(a.cuda(), b.cuda(), block_n=block_n)
    _close(out, _ref(a, b, False, False))


def test_gemm_many_tiles_persistent(cuda_status):
    # more tiles than SMs: exercises the double-buffered accumulators and stage ring wrap-around
    M, N, K = 4096, 4096, 1024
    a, b = _mk((M, K), 5), _mk((N, K), 6)
    out = ops.gemm(a.cuda(), b.cuda())
    _close(out, _ref(a, b, False, False))


def test_gemm_epilogues(cuda_status):
    M, N, K = 300, 264, 192
    a, b = _mk((M, K), 7), _mk((N, K), 8)
    bias, res = _mk((N,), 9), _mk((M, N), 10)
    base = _ref(a, b, False, False)
    # bias + gelu with the pre-activation saved, + residual
    aux = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    out = ops.gemm(a.cuda(), b.cuda(), bias=bias.cuda(), act="gelu", residual=res.cuda(), aux_out=aux)
    pre = (base + bias.float()).to(torch.bfloat16)
    _close(aux, pre.float())
    # the kernel applies GELU to the unrounded fp32 pre-activation
    _close(out, act_reference("gelu", base + bias.float()) + res.float(), family="gemm_act")
    # multiply by gelu'(aux_in)
    out2 = ops.gemm(a.cuda(), b.cuda(), act="dgelu", aux_in=aux)
    _close(out2, base * act_grad_reference("gelu", aux.float().cpu()), family="gemm_act")
    # fp32 output with accumulation and alpha
    acc = torch.ones((M, N), dtype=torch.float32, device="cuda")
    ops.gemm(a.cuda(), b.cuda(), out=acc, accumulate=True, alpha=0.5)
    _close(acc, 1.0 + 0.5 * base)                       # fp32 output: held to 1e-4 relative
    # silu / relu
    out3 = ops.gemm(a.cuda(), b.cuda(), act="silu")
    _close(out3, act_reference("silu", base), family="gemm_act")
    out4 = ops.gemm(a.cuda(), b.cuda(), act="relu")
    _close(out4, torch.relu(base))


def test_linear_autograd_matches_cpu(cuda_status):
    torch.manual_seed(0)
    x = (torch.randn(96, 160) * 0.5).to(torch.bfloat16)
    w = (torch.randn(224, 160) * 0.1).to(torch.bfloat16)
    b = (torch.randn(224) * 0.1).to(torch.bfloat16)
    outs = []
    for dev in ("cpu", "cuda"):
        xd, wd, bd = (t.detach().clone().to(dev).requires_grad_() for t in (x, w, b))
        y = ops.linear(xd, wd, bd, "gelu")
        y.float().sum().backward()
        outs.append((y.float().cpu(), xd.grad.float().cpu(), wd.grad.float().cpu(), bd.grad.float().cpu()))
    for c, g in zip(*outs):
        _close(g, c, family="gemm_act")


@pytest.mark.parametrize("splits", [0, 2, 3, 8])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_split_k_wgrad_shape(splits, out_dtype, cuda_status):
    # weight-gradient shape: small output, long contraction; split-K partial sums are folded in a fixed order
    M, N, K = 768, 264, 8192
    a, b = _mk((K, M), 11), _mk((K, N), 12)
    ref = _ref(a, b, True, True)
    out = torch.full((M, N), 2.0, dtype=out_dtype, device="cuda")
    ops.gemm(a.cuda(), b.cuda(), a_mn=True, b_mn=True, out=out, accumulate=True, splits=splits)
    _close(out, ref + 2.0)
    out2 = torch.full((M, N), 2.0, dtype=out_dtype, device="cuda")
    ops.gemm(a.cuda(), b.cuda(), a_mn=True, b_mn=True, out=out2, accumulate=True, splits=splits)
    assert torch.equal(out, out2)
