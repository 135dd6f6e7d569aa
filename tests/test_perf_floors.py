"""Performance tier (`python -m pytest tests -m perf` on a B200): floors under the headline kernels.

Counterpart of the reference's performance tests (tests/performance/mod.rs; its GPU floor is a 4096^3 matmul above
50 GFLOP/s, tests/performance/gpu.rs:52-59).  The floors here sit about 15 % under what the kernels measure on an
unthrottled B200, so that a regression of a kernel fails the tier while a power-capped run does not.  The tier is not
part of `-m gpu`: timing tests are run on purpose, on a quiet machine.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.perf


def _timed(fn, warmup=3, iters=7):
    from rustral_b200.bench.kernels import timed
    return timed(fn, warmup, iters)          # CUDA events, L2 flushed between iterations, median


def test_gemm_8192_cubed_reaches_1300_tflops():
    from rustral_b200.ops.matmul import gemm
    a = torch.randn(8192, 8192, device="cuda").bfloat16()
    b = (torch.randn(8192, 8192, device="cuda") * 0.02).bfloat16()
    out = torch.empty(8192, 8192, dtype=torch.bfloat16, device="cuda")
    ms = _timed(lambda: gemm(a, b, out=out))
    tflops = 2.0 * 8192 ** 3 / ms / 1e9
    assert tflops >= 1300, f"{tflops:.0f} TFLOP/s"


def test_cross_entropy_streams_5_tb_per_s():
    from rustral_b200 import ops
    rows, n = 32768, 50304
    logits = torch.randn(rows, n, device="cuda").bfloat16()
    tgt = torch.randint(0, 50257, (rows,), device="cuda")
    ms = _timed(lambda: ops.cross_entropy_fwd_bwd(logits, tgt, 50257, 1.0, dlogits=logits), iters=5)
    tbs = 3.0 * rows * n * 2 / ms / 1e9          # the row is read twice and written once
    assert tbs >= 5.0, f"{tbs:.2f} TB/s"


def test_paged_decode_attention_streams_4_tb_per_s():
    from rustral_b200.bench import kernels as K
    out = K.main(["paged", "--batch", "64", "--context", "4096"])
    assert out["gbs"] >= 4000, out


def test_attention_forward_floors():
    from rustral_b200.ops import attention as A
    for (B, S, H, Hk, D), floor in (((32, 1024, 12, 12, 64), 250), ((4, 4096, 32, 8, 128), 700)):
        q = torch.randn(B, S, H, D, device="cuda").bfloat16()
        k = torch.randn(B, S, Hk, D, device="cuda").bfloat16()
        v = torch.randn(B, S, Hk, D, device="cuda").bfloat16()
        o = torch.empty_like(q)
        ms = _timed(lambda: A.attention_forward(q, k, v, True, 1 / math.sqrt(D), out=o))
        tflops = 4.0 * B * H * S * S * D / 2 / ms / 1e9
        assert tflops >= floor, f"head dim {D}: {tflops:.0f} TFLOP/s < {floor}"


def test_norm_backward_streams_3_tb_per_s():
    from rustral_b200.bench import kernels as K
    out = K.main(["norm", "--rows", "32768", "--n", "768", "--backward"])
    assert out["gbs"] >= 3000, out
