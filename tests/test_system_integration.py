"""System suite, integration category (the reference's tests/integration/mod.rs: core -> nn, autodiff, optimiser,
data -> nn, sequential chaining, mixed precision, save / load, backend consistency, parameter sharing, mode switching),
one test per case, on the CPU reference backend."""
import math

import pytest
import torch

from rustral_b200 import ops
from rustral_b200.core import CpuBackend, ForwardCtx
from rustral_b200.nn import (CrossEntropyLoss, Dropout, DropoutConfig, Embedding, EmbeddingConfig, LayerNorm, LinearBuilder,
                             MSELoss, Sequential, TransformerEncoder, TransformerEncoderConfig)
from rustral_b200.nn.sequential import chain
from rustral_b200.optim import Adam, Sgd
from rustral_b200.runtime.model_io import load_model, save_model

BE = CpuBackend()
T = BE.ops()


def test_core_to_nn_integration():
    """Tensors made by the backend's op table flow through layers and back into op-table calls."""
    x = T.tensor_from_vec([float(i) for i in range(12)], (3, 4))
    lin = LinearBuilder(4, 2).with_bias().seed(1).build(BE)
    y = lin(x)
    assert y.shape == (3, 2)
    manual = T.add_row_vector(T.matmul(x, T.transpose(lin.weight.tensor.detach())), lin.bias.tensor.detach())
    assert torch.allclose(y.detach(), manual, atol=1e-6)
    assert T.tensor_to_vec(T.relu(T.tensor_from_vec([-1.0, 2.0], (1, 2)))) == [0.0, 2.0]


def test_autodiff_integration():
    """A two-layer network's gradients equal the hand-derived ones."""
    a = LinearBuilder(3, 4).seed(2).build(BE)
    b = LinearBuilder(4, 1).seed(3).build(BE)
    x = torch.randn(5, 3, generator=torch.Generator().manual_seed(4))
    ctx = ForwardCtx.train(BE)
    h = torch.relu(a(x, ctx))
    loss = b(h, ctx).sum()
    loss.backward()
    gb = h.detach().sum(0, keepdim=True)                       # d loss / d W_b = sum_i h_i
    assert torch.allclose(b.weight.tensor.grad, gb, atol=1e-6)
    mask = (a(x, ctx).detach() > 0).float()
    ga = (mask * b.weight.tensor.detach()).t() @ x             # d loss / d W_a
    assert torch.allclose(a.weight.tensor.grad, ga, atol=1e-5)


def test_optim_integration():
    """Adam drives a linear regression to its solution; SGD with momentum reduces the loss monotonically at a small rate."""
    g = torch.Generator().manual_seed(5)
    w_true = torch.randn(4, 1, generator=g)
    x = torch.randn(64, 4, generator=g)
    y = x @ w_true
    lin = LinearBuilder(4, 1).seed(6).build(BE)
    opt = Adam(0.05)
    ctx = ForwardCtx.train(BE)
    for _ in range(300):
        lin.zero_grad()
        MSELoss()(lin(x, ctx), y).backward()
        opt.step(lin.parameters())
    assert torch.allclose(lin.weight.tensor.detach().t(), w_true, atol=2e-2)
    lin2 = LinearBuilder(4, 1).seed(7).build(BE)
    sgd, losses = Sgd(0.01, momentum=0.5), []
    for _ in range(30):
        lin2.zero_grad()
        l = MSELoss()(lin2(x, ctx), y)
        l.backward()
        sgd.step(lin2.parameters())
        losses.append(float(l))
    assert all(b <= a + 1e-7 for a, b in zip(losses, losses[1:])) and losses[-1] < 0.7 * losses[0]


def test_data_nn_integration():
    """Batches from the data loader feed an embedding + classifier; one epoch visits every example exactly once."""
    from rustral_b200.data import simple_loader
    examples = [([i % 7, (i * 3) % 7, (i * 5) % 7], i % 2) for i in range(20)]
    loader = simple_loader(examples, batch_size=6)
    emb = Embedding.new(BE, 7, 8)
    head = LinearBuilder(8, 2).with_bias().build(BE)
    ctx = ForwardCtx.train(BE)
    seen = 0
    for batch in loader:
        ids = torch.tensor([ex[0] for ex in batch])
        labels = torch.tensor([ex[1] for ex in batch])
        logits = head(emb(ids, ctx).mean(1), ctx)
        loss = CrossEntropyLoss()(logits, labels)
        assert logits.shape == (len(batch), 2) and math.isfinite(float(loss))
        seen += len(batch)
    assert seen == 20


def test_sequential_chaining():
    l1, l2, l3 = (LinearBuilder(4, 4).with_bias().seed(s).build(BE) for s in (1, 2, 3))
    x = torch.randn(2, 4, generator=torch.Generator().manual_seed(8))
    ctx = ForwardCtx.inference(BE)
    seq = Sequential(l1, l2, l3)
    assert torch.equal(seq(x, ctx), l3(l2(l1(x, ctx), ctx), ctx))
    assert torch.equal(chain(chain(l1, l2), l3)(x, ctx), seq(x, ctx))
    names = [n for n, _ in seq.named_parameters()]
    assert names == ["layers.0.weight", "layers.0.bias", "layers.1.weight", "layers.1.bias", "layers.2.weight", "layers.2.bias"]


def test_mixed_precision_integration():
    """bf16 activations through fp32-parameter layers stay within bf16 rounding of the fp32 result."""
    lin = LinearBuilder(64, 32).with_bias().seed(9).build(BE)
    x = torch.randn(16, 64, generator=torch.Generator().manual_seed(10))
    ref = lin(x)
    low = ops.linear(x.bfloat16(), lin.weight.tensor.detach().bfloat16(), lin.bias.tensor.detach().bfloat16())
    assert low.dtype == torch.bfloat16
    assert float((low.float() - ref).abs().max()) < 0.05 * float(ref.abs().max())
    from rustral_b200.optim import MixedPrecisionOptimizer
    p = LinearBuilder(8, 8).seed(11).build(BE)
    from rustral_b200.optim import LossScaleScheduler
    mp = MixedPrecisionOptimizer(Adam(1e-2), loss_scale=LossScaleScheduler(1024.0))
    p.zero_grad()
    mp.scale_loss(p(torch.ones(2, 8), ForwardCtx.train(BE)).sum()).backward()
    before = p.weight.tensor.detach().clone()
    assert mp.step(p.parameters()) and not torch.equal(before, p.weight.tensor.detach())


def test_save_load_integration():
    cfg = TransformerEncoderConfig(32, 4, 2, 64, 0.0, 16)
    a, b = TransformerEncoder.new(BE, cfg, 50, seed=1), TransformerEncoder.new(BE, cfg, 50, seed=2)
    ids = [[1, 2, 3, 4], [5, 6, 7, 8]]
    ctx = ForwardCtx.inference(BE)
    assert not torch.equal(a.forward(ids, ctx), b.forward(ids, ctx))
    load_model(b, save_model(a))
    assert torch.equal(a.forward(ids, ctx), b.forward(ids, ctx))
    assert [n for n, _ in a.named_parameters()] == [n for n, _ in b.named_parameters()]


def test_backend_consistency():
    """The C++ oracle, the op table and plain PyTorch agree on the same inputs."""
    from rustral_b200.ops import oracle
    g = torch.Generator().manual_seed(12)
    a, b = torch.randn(7, 5, generator=g), torch.randn(5, 3, generator=g)
    want = a @ b
    assert torch.allclose(T.matmul(a, b), want, atol=1e-6)
    assert torch.allclose(oracle.matmul(a, b), want, atol=1e-5)
    x = torch.randn(1, 9, generator=g)       # the op table's softmax normalises over the whole tensor, as the reference's does
    assert torch.allclose(T.softmax(x), torch.softmax(x, -1), atol=1e-6)
    assert torch.allclose(oracle.softmax_rows(torch.randn(4, 9, generator=g)).sum(-1), torch.ones(4), atol=1e-6)
    assert torch.allclose(oracle.softmax_rows(x), torch.softmax(x, -1), atol=1e-6)


def test_parameter_sharing():
    """One layer used twice accumulates both uses' gradients into the same parameter and lists it once."""
    shared = LinearBuilder(4, 4).seed(13).build(BE)
    x = torch.randn(3, 4, generator=torch.Generator().manual_seed(14))
    ctx = ForwardCtx.train(BE)
    shared(shared(x, ctx), ctx).sum().backward()
    both = shared.weight.tensor.grad.clone()
    shared.zero_grad()
    w = shared.weight.tensor.detach()
    h = (x @ w.t()).detach()
    first = torch.ones(3, 4) @ w                                      # gradient reaching the first use's output
    want = torch.ones(3, 4).t() @ h + first.t() @ x
    assert torch.allclose(both, want, atol=1e-5)
    seq = Sequential(shared, shared)
    ids = {id(p.tensor) for p in seq.parameters()}
    assert len(ids) == 1


def test_mode_switching():
    drop = Dropout(DropoutConfig(0.5))
    x = torch.ones(64, 64)
    tr, inf = ForwardCtx.train(BE), ForwardCtx.inference(BE)
    y_train = drop(x, tr)
    assert torch.equal(drop(x, inf), x)
    kept = (y_train != 0).float().mean()
    assert 0.35 < float(kept) < 0.65 and torch.allclose(y_train[y_train != 0], torch.full_like(y_train[y_train != 0], 2.0))
    assert torch.equal(drop(x, inf), x)                                  # back to inference: identity again
    ln = LayerNorm.new(BE, 64)
    assert torch.equal(ln(x, tr), ln(x, inf))                            # mode-independent layers agree in both modes
