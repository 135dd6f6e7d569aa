"""Golden numerics: the CPU reference path and the C++ oracle against the same operations evaluated in float64
(crates/core/tests/golden_microblock_ops.rs with tests/golden/mod.rs; tolerances of tests/common/numeric.rs for the CPU
backend: 1e-5 relative, 1e-6 absolute, looser only where the operation amplifies rounding)."""
import math

import pytest
import torch

from rustral_b200 import ops
from rustral_b200.ops import oracle


def _r(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def _close(got, want64, rtol=1e-5, atol=1e-6):
    got, want = got.double(), want64.double()
    assert got.shape == want.shape
    excess = (got - want).abs() - (atol + rtol * want.abs())
    assert float(excess.max()) <= 0, f"max excess {float(excess.max()):.3g} at {int(excess.argmax())}"


@pytest.mark.parametrize("rows,cols,scale", [(4, 7, 1.0), (3, 1000, 5.0), (2, 64, 50.0)])
def test_softmax_and_log_softmax(rows, cols, scale):
    x = _r(rows, cols, seed=rows, scale=scale)
    want = torch.softmax(x.double(), -1)
    _close(ops.softmax(x), want)
    _close(oracle.softmax_rows(x), want)
    _close(ops.log_softmax(x), torch.log_softmax(x.double(), -1), atol=1e-5)
    assert torch.allclose(ops.softmax(x).sum(-1), torch.ones(rows), atol=1e-6)


@pytest.mark.parametrize("n", [8, 96, 1024])
def test_layer_norm_and_rms_norm(n):
    x = _r(5, n, seed=n, scale=3.0) + 2.0
    g, b = _r(n, seed=1), _r(n, seed=2)
    xd = x.double()
    mean, var = xd.mean(-1, keepdim=True), xd.var(-1, unbiased=False, keepdim=True)
    want = (xd - mean) / torch.sqrt(var + 1e-5) * g.double() + b.double()
    _close(ops.layer_norm(x, g, b, 1e-5), want, rtol=2e-5, atol=5e-6)
    _close(oracle.layer_norm(x, g, b, 1e-5)[0], want, rtol=2e-5, atol=5e-6)         # the oracle also returns mean and rstd
    want_r = xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + 1e-5) * g.double()
    _close(ops.rms_norm(x, g, 1e-5), want_r, rtol=2e-5, atol=5e-6)


def test_activations():
    x = torch.linspace(-8, 8, 4001)
    xd = x.double()
    gelu = 0.5 * xd * (1 + torch.tanh(math.sqrt(2 / math.pi) * (xd + 0.044715 * xd ** 3)))
    _close(ops.gelu(x), gelu)
    _close(ops.silu(x), xd * torch.sigmoid(xd))
    _close(ops.relu(x), torch.relu(xd), rtol=0, atol=0)
    _close(oracle.unary("gelu", x), gelu)
    # derivatives through autograd against the analytic float64 derivative
    xg = x.clone().requires_grad_()
    ops.gelu(xg).sum().backward()
    t = torch.tanh(math.sqrt(2 / math.pi) * (xd + 0.044715 * xd ** 3))
    dgelu = 0.5 * (1 + t) + 0.5 * xd * (1 - t * t) * math.sqrt(2 / math.pi) * (1 + 3 * 0.044715 * xd * xd)
    _close(xg.grad, dgelu, rtol=1e-5, atol=1e-6)


def test_cross_entropy_loss_and_gradient():
    logits, tgt = _r(9, 50, seed=3, scale=4.0), torch.tensor([0, 49, 7, 7, 12, -100, 3, 30, 1])
    ld = logits.double()
    valid = tgt != -100
    lse = torch.logsumexp(ld, -1)
    want = (lse - ld.gather(1, tgt.clamp_min(0)[:, None])[:, 0])[valid].mean()
    lg = logits.clone().requires_grad_()
    loss = ops.cross_entropy(lg, tgt)
    _close(loss.detach(), want)
    loss.backward()
    p = torch.softmax(ld, -1)
    p[torch.arange(9), tgt.clamp_min(0)] -= 1.0
    p[~valid] = 0.0
    _close(lg.grad, p / int(valid.sum()), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("causal", [False, True])
def test_attention(causal):
    q, k, v = _r(2, 9, 4, 16, seed=4), _r(2, 9, 2, 16, seed=5), _r(2, 9, 2, 16, seed=6)
    qd, kd, vd = (t.double().permute(0, 2, 1, 3) for t in (q, k, v))
    kd, vd = kd.repeat_interleave(2, 1), vd.repeat_interleave(2, 1)
    s = qd @ kd.transpose(-1, -2) / 4.0
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(9, 9, dtype=torch.bool), 1), float("-inf"))
    want = (torch.softmax(s, -1) @ vd).permute(0, 2, 1, 3)
    _close(ops.flash_attention(q, k, v, causal), want, rtol=2e-5, atol=2e-6)
    _close(oracle.attention(q, k, v, causal, 0.25), want, rtol=2e-5, atol=2e-6)


def test_matmul_and_linear_epilogues():
    a, w, b, res = _r(17, 33, seed=7), _r(21, 33, seed=8), _r(21, seed=9), _r(17, 21, seed=10)
    base = a.double() @ w.double().t()
    _close(ops.gemm(a, w), base, rtol=1e-5, atol=1e-5)
    _close(oracle.matmul(a, w.t().contiguous()), base, rtol=1e-5, atol=1e-5)
    pre = base + b.double()
    gelu = 0.5 * pre * (1 + torch.tanh(math.sqrt(2 / math.pi) * (pre + 0.044715 * pre ** 3)))
    _close(ops.linear(a, w, b, "gelu", res), gelu + res.double(), rtol=1e-5, atol=1e-5)
    _close(oracle.linear(a, w, b, "gelu"), gelu, rtol=1e-5, atol=1e-5)
    _close(ops.gemm(a.t().contiguous(), w.t().contiguous(), a_mn=True, b_mn=True, alpha=0.5), 0.5 * base, rtol=1e-5, atol=1e-5)


def test_adam_update_against_the_float64_recurrence():
    p0, g = _r(1000, seed=11), _r(1000, seed=12)
    p, m, v = p0.clone(), torch.zeros(1000), torch.zeros(1000)
    pd, md, vd = p0.double(), torch.zeros(1000, dtype=torch.float64), torch.zeros(1000, dtype=torch.float64)
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.999, 1e-8, 0.1
    for t in range(1, 6):
        gt = g * (1.0 + 0.1 * t)
        ops.adam_step(p, m, v, gt, lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd, step=t, decoupled=True)
        gd = gt.double()
        md = b1 * md + (1 - b1) * gd
        vd = b2 * vd + (1 - b2) * gd * gd
        pd = pd - lr * ((md / (1 - b1 ** t)) / (torch.sqrt(vd / (1 - b2 ** t)) + eps) + wd * pd)
    _close(p, pd, rtol=1e-5, atol=1e-6)
    _close(m, md)
    _close(v, vd)
