"""Training-path kernels of the recurrent cells, Conv2d and expert-choice routing against the same modules on the CPU
reference backend in fp32 (parameters and inputs rounded to bf16 on both sides)."""
import pytest
import torch

from rustral_b200.core import CpuBackend, ForwardCtx
from rustral_b200.nn import Conv2d, Conv2dConfig, ExpertChoiceConfig, ExpertChoiceRouter, GruCell, LstmCell
from rustral_b200.nn.expert_choice import ec_select, ec_table
from tolerances import assert_close

pytestmark = pytest.mark.gpu
BE = CpuBackend()


def _to_cuda_bf16(cell):
    for name in ("wx", "wh", "b", "weight", "bias", "router"):
        p = getattr(cell, name, None)
        if p is not None:
            p.tensor = p.tensor.detach().bfloat16().cuda().requires_grad_()
    return cell


def _round_params(cell):
    for name in ("wx", "wh", "b", "weight", "bias", "router"):
        p = getattr(cell, name, None)
        if p is not None:
            p.tensor = p.tensor.detach().bfloat16().float().requires_grad_()
    return cell


@pytest.mark.parametrize("cls", [LstmCell, GruCell])
@pytest.mark.parametrize("T,B,I,H", [(6, 4, 32, 64), (3, 5, 24, 40)])
def test_recurrent_cells_train_on_the_gate_kernels(cls, T, B, I, H, cuda_status):
    ref, dev = _round_params(cls.new(BE, I, H, seed=3)), _to_cuda_bf16(cls.new(BE, I, H, seed=3))
    g = torch.Generator().manual_seed(T * 100 + B)
    xs = torch.randn(T, B, I, generator=g).bfloat16()
    w = torch.randn(T, B, H, generator=g).bfloat16()
    ctx = ForwardCtx.train(BE)
    xr = xs.float().requires_grad_()
    out_r, _ = ref.forward_sequence(xr, ctx)
    (out_r * w.float()).sum().backward()
    xd = xs.cuda().requires_grad_()
    out_d, _ = dev.forward_sequence(xd, ctx)
    (out_d.float() * w.cuda().float()).sum().backward()
    assert out_d.dtype == torch.bfloat16
    assert_close(out_d, out_r, "norm", "hidden states")
    assert_close(xd.grad, xr.grad, "attention_grad", "dx")
    for name in ("wx", "wh", "b"):
        assert_close(getattr(dev, name).tensor.grad, getattr(ref, name).tensor.grad, "attention_grad", f"d{name}")


@pytest.mark.parametrize("N,C,H,W,O,k,stride,nopad", [(2, 3, 16, 16, 8, 3, 1, False), (2, 3, 17, 23, 13, 3, 2, False),
                                                      (1, 8, 12, 12, 16, 5, 1, True), (3, 1, 28, 28, 6, 3, 1, False)])
def test_conv2d_trains_on_im2col_gemm_col2im_kernels(N, C, H, W, O, k, stride, nopad, cuda_status):
    conv = Conv2d.new(BE, Conv2dConfig(O, k, k, stride=stride, no_padding=nopad, in_channels=C), seed=5)
    g = torch.Generator().manual_seed(N * 10 + C)
    with torch.no_grad():
        conv.bias.tensor.copy_(torch.randn(O, generator=g) * 0.1)
    x = torch.randn(N, C, H, W, generator=g).bfloat16()
    wt, bs = conv.weight.tensor.detach().bfloat16(), conv.bias.tensor.detach().bfloat16()
    pad = 0 if nopad else k // 2
    xr, wr, br = x.float().requires_grad_(), wt.float().requires_grad_(), bs.float().requires_grad_()
    yr = torch.nn.functional.conv2d(xr, wr, br, stride=stride, padding=pad)
    dy = torch.randn(yr.shape, generator=g).bfloat16()
    yr.backward(dy.float())
    _to_cuda_bf16(conv)
    xd = x.cuda().requires_grad_()
    yd = conv(xd, ForwardCtx.train(BE))
    assert yd.shape == yr.shape and yd.dtype == torch.bfloat16
    yd.backward(dy.cuda())
    assert_close(yd, yr, "gemm_bf16", "conv output")
    assert_close(xd.grad, xr.grad, "attention_grad", "conv dx")
    assert_close(conv.weight.tensor.grad, wr.grad, "attention_grad", "conv dW")
    assert_close(conv.bias.tensor.grad, br.grad, "attention_grad", "conv db")
    # the same call twice gives the same bits (no atomics in col2im or in the reductions)
    xd2 = x.cuda().requires_grad_()
    conv.weight.tensor.grad = None
    conv(xd2, ForwardCtx.train(BE)).backward(dy.cuda())
    assert torch.equal(xd2.grad, xd.grad)


@pytest.mark.parametrize("T,E,cap", [(64, 4, 8), (1000, 8, 100), (4096, 16, 256), (33, 3, 33)])
def test_expert_choice_selection_and_table(T, E, cap, cuda_status):
    g = torch.Generator().manual_seed(T + E)
    probs = torch.softmax(torch.randn(T, E, generator=g), -1)
    probs[::7] = probs[0]                                    # exact ties across tokens
    idx_r, gate_r = ec_select(probs, cap)
    idx_d, gate_d = ec_select(probs.cuda(), cap)
    assert torch.equal(idx_d.cpu(), idx_r) and torch.equal(gate_d.cpu(), gate_r)
    assert torch.equal(ec_table(idx_d, T).cpu(), ec_table(idx_r, T))


def test_expert_choice_router_trains_on_native_kernels(cuda_status):
    d, E, T = 64, 4, 96
    cfg = ExpertChoiceConfig(d, E, 128, tokens_per_expert=24)
    ref, dev = _round_params(ExpertChoiceRouter.new(BE, cfg, seed=9)), _to_cuda_bf16(ExpertChoiceRouter.new(BE, cfg, seed=9))
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        big = (torch.randn(E, d, generator=g) * 0.5).bfloat16()
        ref.router.tensor.copy_(big.float()); dev.router.tensor.copy_(big.cuda())
    ws = [(torch.randn(d, d, generator=g) * 0.1).bfloat16() for _ in range(E)]
    x = torch.randn(T, d, generator=g).bfloat16()
    dy = torch.randn(T, d, generator=g).bfloat16()
    xr = x.float().requires_grad_()
    wr = [w.float().requires_grad_() for w in ws]
    yr = ref.forward(xr, lambda e, rows: rows @ wr[e].t(), ForwardCtx.train(BE))
    yr.backward(dy.float())
    from rustral_b200 import ops
    xd = x.cuda().requires_grad_()
    wd = [w.cuda().requires_grad_() for w in ws]
    yd = dev.forward(xd, lambda e, rows: ops.linear(rows, wd[e]), ForwardCtx.train(BE))
    yd.backward(dy.cuda())
    assert dev.last_stats.unrouted_tokens == ref.last_stats.unrouted_tokens
    assert_close(yd, yr, "attention", "expert-choice output")
    assert_close(xd.grad, xr.grad, "attention_grad", "dx")
    assert_close(dev.router.tensor.grad, ref.router.tensor.grad, "attention_grad", "drouter")
    for e in range(E):
        assert_close(wd[e].grad, wr[e].grad, "attention_grad", f"dW{e}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,W,k,stride", [(8, 8, 2, 2), (9, 11, 3, 2), (7, 7, 3, 1), (6, 6, 6, 6)])
def test_max_pool2d_forward_and_backward(H, W, k, stride, dtype, cuda_status):
    from rustral_b200.nn.conv import global_max_pool2d, max_pool2d
    g = torch.Generator().manual_seed(H * 10 + k)
    x = torch.randn(3, 4, H, W, generator=g).to(dtype)
    xr = x.float().clone().requires_grad_()            # a copy: for fp32 `x.float()` is x itself
    yr = torch.nn.functional.max_pool2d(xr, k, stride)
    dy = torch.randn(yr.shape, generator=g).to(dtype)
    yr.backward(dy.float())
    xd = x.detach().cuda().requires_grad_()
    yd = max_pool2d(xd, k, stride)
    yd.backward(dy.cuda())
    assert torch.equal(yd.float().cpu(), yr.detach().to(dtype).float())
    assert torch.allclose(xd.grad.float().cpu(), xr.grad, atol=2e-2 if dtype is torch.bfloat16 else 1e-6)
    if H == W:
        assert torch.equal(global_max_pool2d(x.cuda()).float().cpu(), x.float().amax((2, 3)))
