"""8-bit tensor-core GEMM (tcgen05 kind::f8f6f4) and the quantisation kernels against fp32 restatements of the same
arithmetic: the e4m3 / e5m2 operands are exact in fp32, so the only differences are accumulation order and the output
rounding."""
import pytest
import torch

from rustral_b200 import ops
from rustral_b200.ops import quant as Q
from tolerances import assert_close

pytestmark = pytest.mark.gpu


def _bytes(shape, seed, dtype=torch.float8_e4m3fn, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).view(torch.uint8)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 256, 256), (130, 72, 144), (1000, 768, 784), (64, 64, 64), (8, 16, 16),
                                   (2048, 2304, 768), (512, 4096, 4096)])
@pytest.mark.parametrize("block_n", [0, 64, 128, 192, 256])
def test_fp8_gemm_matches_fp32_product_of_the_same_bytes(M, N, K, block_n, cuda_status):
    a8, b8 = _bytes((M, K), 1), _bytes((N, K), 2)
    ref = a8.view(torch.float8_e4m3fn).float() @ b8.view(torch.float8_e4m3fn).float().t()
    out = Q.gemm_fp8(a8.cuda(), None, b8.cuda(), None, out_dtype=torch.float32, block_n=block_n)
    assert_close(out, ref, "gemm_f32", f"fp8 {M}x{N}x{K} bn{block_n}")
    out2 = Q.gemm_fp8(a8.cuda(), None, b8.cuda(), None, out_dtype=torch.float32, block_n=block_n)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("act", ["none", "gelu"])
@pytest.mark.parametrize("b_e5m2", [False, True])
def test_fp8_gemm_scales_bias_and_activation_in_the_epilogue(act, b_e5m2, cuda_status):
    M, N, K = 300, 200, 256
    a8 = _bytes((M, K), 3)
    b8 = _bytes((N, K), 4, torch.float8_e5m2 if b_e5m2 else torch.float8_e4m3fn)
    g = torch.Generator().manual_seed(5)
    sa = torch.rand(M, generator=g) * 0.1 + 0.01
    sb = torch.rand(N, generator=g) * 0.1 + 0.01
    bias = (torch.randn(N, generator=g) * 0.1).bfloat16()
    res = (torch.randn(M, N, generator=g) * 0.1).bfloat16()
    ref = Q.gemm_fp8(a8, sa, b8, sb, bias=bias, act=act, residual=res, out_dtype=torch.float32, b_e5m2=b_e5m2)
    out = Q.gemm_fp8(a8.cuda(), sa.cuda(), b8.cuda(), sb.cuda(), bias=bias.cuda(), act=act, residual=res.cuda(), b_e5m2=b_e5m2)
    assert out.dtype == torch.bfloat16
    assert_close(out, ref, "gemm_act" if act == "gelu" else "gemm_bf16", f"fp8 epilogue {act}")


@pytest.mark.parametrize("rows,n", [(7, 64), (33, 768), (128, 1024), (5, 4096), (3, 8192), (1, 16)])
def test_fp8_row_quantiser_matches_the_reference_rounding(rows, n, cuda_status):
    g = torch.Generator().manual_seed(rows * 1000 + n)
    x = (torch.randn(rows, n, generator=g) * torch.rand(rows, 1, generator=g) * 4).bfloat16()
    x[0, : n // 2] = 0
    q_ref, s_ref = Q.quantize_fp8_rows(x)
    q, s = Q.quantize_fp8_rows(x.cuda())
    assert torch.equal(s.cpu(), s_ref) and torch.equal(q.cpu(), q_ref)       # same scale, same reciprocal, same rounding
    a = q.cpu().view(torch.float8_e4m3fn).float()
    back = a * s.cpu()[:, None]
    assert float((back - x.float()).abs().max()) <= float(x.float().abs().max()) * 2 ** -4
    zq, zs = Q.quantize_fp8_rows(torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda"))
    assert not zq.any() and torch.equal(zs.cpu(), torch.ones(4))


def test_int8_and_int4_expansion_are_exact(cuda_status):
    g = torch.Generator().manual_seed(9)
    q = torch.randint(-128, 128, (37, 208), generator=g, dtype=torch.int8)
    assert torch.equal(Q.dequant_int8(q.cuda()).cpu(), q.float().bfloat16())
    zp = torch.randint(-20, 20, (37,), generator=g).float()
    assert torch.equal(Q.dequant_int8(q.cuda(), zp.cuda()).cpu(), (q.float() - zp[:, None]).bfloat16())
    assert torch.equal(Q.dequant_int8(q.cuda(), zp[:1].cuda()).cpu(), (q.float() - zp[0]).bfloat16())
    packed = torch.randint(0, 256, (19, 96), generator=g, dtype=torch.uint8)
    scales = torch.rand(19, 3, generator=g) * 0.1
    assert torch.equal(Q.dequant_int4(packed.cuda(), scales.cuda(), 64).cpu(), Q.dequant_int4(packed, scales, 64))


@pytest.mark.parametrize("scheme", ["int8", "int8_asymmetric", "int8_per_channel", "fp8_e4m3", "fp8_e5m2", "int4"])
def test_quantized_layers_on_the_gpu_match_their_cpu_definition(scheme, cuda_status):
    from rustral_b200.core import CpuBackend
    from rustral_b200.nn import GPTQLinear, LinearBuilder, QuantizationScheme, QuantizedLinear
    torch.manual_seed(0)
    lin = LinearBuilder(256, 48).with_bias().build(CpuBackend())
    with torch.no_grad():
        lin.weight.tensor.copy_(torch.randn(48, 256) * 0.1)
        lin.bias.tensor.copy_(torch.randn(48) * 0.1)
    q = GPTQLinear.from_linear(lin, 64) if scheme == "int4" else QuantizedLinear.from_linear(lin, QuantizationScheme(scheme))
    x = torch.randn(3, 10, 256).bfloat16()
    if scheme == "int4":       # the GPU path multiplies by the bf16-rounded expansion of the nibbles
        ref = x.float() @ Q.dequant_int4(q.packed, q.scales, q.group_size).float().t() + lin.bias.tensor
    else:
        ref = q(x.float())
    for name, v in list(vars(q).items()):
        if isinstance(v, torch.Tensor):
            setattr(q, name, v.cuda())
    if hasattr(q, "params"):
        q.params.scale, q.params.zero_point = q.params.scale.cuda(), q.params.zero_point.cuda()
    out = q(x.cuda())
    assert out.shape == (3, 10, 48) and out.dtype == torch.bfloat16
    assert_close(out, ref, "gemm_bf16", scheme)
