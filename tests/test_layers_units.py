"""Basic layers against their formulas (crates/nn/src/{linear,embedding,normalization,dropout,loss,sequential}.rs
`mod tests`), on the CPU reference backend."""
import math

import pytest
import torch
import torch.nn.functional as F

from rustral_b200.core import CpuBackend, ForwardCtx, InvalidArgument, ShapeMismatch
from rustral_b200.nn import (BCEWithLogitsLoss, CrossEntropyLoss, Dropout, DropoutConfig, Embedding, LayerNorm, Linear, LinearBuilder,
                             LinearGELU, LinearReLU, LinearSiLU, MSELoss, RMSNorm, Sequential, Sequential2, chain)
from rustral_b200.symbolic import Vocabulary

BE = CpuBackend()
INF, TRAIN = ForwardCtx.inference(BE), ForwardCtx.train(BE, seed=11)


def _x(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


# ---- linear ---------------------------------------------------------------------------------------------------------
def test_linear_builder_options():
    plain = LinearBuilder(6, 4).build(BE)
    assert plain.bias is None and plain.weight.shape == (4, 6) and [n for n, _ in plain.named_parameters()] == ["weight"]
    a, b = LinearBuilder(6, 4).with_bias().seed(3).build(BE), LinearBuilder(6, 4).with_bias().seed(3).build(BE)
    assert torch.equal(a.weight.tensor, b.weight.tensor) and torch.equal(a.bias.tensor, b.bias.tensor)      # seeded
    assert not torch.equal(a.weight.tensor, LinearBuilder(6, 4).seed(4).build(BE).weight.tensor)
    wide = LinearBuilder(512, 512).seed(1).scale(0.5).build(BE)
    assert float(wide.weight.tensor.std()) == pytest.approx(0.5, rel=0.02) and abs(float(wide.weight.tensor.mean())) < 0.01
    z = LinearBuilder(6, 4).with_bias().zero_bias().build(BE)
    assert float(z.bias.tensor.abs().sum()) == 0.0 and z.bias.tensor.requires_grad
    for bad in ((0, 4), (4, -1)):
        with pytest.raises(InvalidArgument):
            LinearBuilder(*bad)
    with pytest.raises(InvalidArgument):
        LinearBuilder(4, 4).activation("relu").build(BE)             # the fused activations need a bias
    assert Linear.new(BE, 3, 2, bias=False).bias is None


@pytest.mark.parametrize("name,cls,fn", [("relu", LinearReLU, torch.relu), ("gelu", LinearGELU, lambda t: F.gelu(t, approximate="tanh")),
                                         ("silu", LinearSiLU, F.silu)])
def test_fused_activation_linears_equal_linear_then_activation(name, cls, fn):
    lin = LinearBuilder(8, 5).with_bias().seed(2).activation(name).build(BE)
    assert isinstance(lin, cls) and lin.activation == name
    x = _x(3, 7, 8)
    want = fn(x @ lin.weight.tensor.t() + lin.bias.tensor)
    assert torch.allclose(lin(x, INF), want, atol=1e-6)
    xg = x.clone().requires_grad_()
    lin(xg, TRAIN).sum().backward()
    xr = x.clone().requires_grad_()
    fn(xr @ lin.weight.tensor.detach().t() + lin.bias.tensor.detach()).sum().backward()
    assert torch.allclose(xg.grad, xr.grad, atol=1e-5)


def test_linear_residual_is_added_after_the_activation():
    lin = LinearBuilder(4, 4).with_bias().activation("relu").build(BE)
    x, r = _x(2, 4), _x(2, 4, seed=1)
    assert torch.allclose(lin(x, INF, r), torch.relu(x @ lin.weight.tensor.t() + lin.bias.tensor) + r, atol=1e-6)


# ---- embedding ------------------------------------------------------------------------------------------------------
def test_embedding_gathers_rows_accumulates_repeated_ids_and_checks_the_range():
    emb = Embedding.new(BE, 10, 4, seed=1)
    ids = torch.tensor([[1, 3, 3], [9, 0, 3]])
    out = emb(ids, TRAIN)
    assert out.shape == (2, 3, 4) and torch.equal(out[0, 1], emb.embed.tensor[3].detach())
    out.sum().backward()
    g = emb.embed.tensor.grad
    assert g[3].tolist() == [3.0] * 4 and g[1].tolist() == [1.0] * 4 and g[2].abs().sum() == 0     # id 3 was used three times
    for bad in ([[10]], [[-1]]):
        with pytest.raises(InvalidArgument):
            emb(torch.tensor(bad), INF)
    assert emb(torch.zeros(0, dtype=torch.int64), INF).shape == (0, 4)
    vocab = Vocabulary.with_specials("<unk>", ["cat", "dog"])
    e2 = Embedding.new(BE, len(vocab), 4, vocab=vocab)
    assert torch.equal(e2.lookup("dog")[0], e2.embed.tensor[2].detach()) and torch.equal(e2.lookup("bird")[0], e2.embed.tensor[0].detach())
    with pytest.raises(InvalidArgument):
        emb.lookup("cat")
    assert [n for n, _ in emb.named_parameters()] == ["embed"]


# ---- normalisation --------------------------------------------------------------------------------------------------
def test_layer_norm_and_rms_norm_formulas_and_gradients():
    x = _x(4, 6, 16) * 3 + 1
    ln = LayerNorm.new(BE, 16)
    with torch.no_grad():
        ln.weight.tensor.copy_(_x(16, seed=2)); ln.bias.tensor.copy_(_x(16, seed=3))
    want = F.layer_norm(x, (16,), ln.weight.tensor, ln.bias.tensor, 1e-5)
    assert torch.allclose(ln(x, INF), want, atol=1e-5)
    y = LayerNorm.new(BE, 16)(x, INF)
    assert torch.allclose(y.mean(-1), torch.zeros(4, 6), atol=1e-5) and torch.allclose(y.var(-1, unbiased=False), torch.ones(4, 6), atol=1e-3)
    rms = RMSNorm.new(BE, 16, eps=1e-6)
    want_r = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * rms.weight.tensor
    assert torch.allclose(rms(x, INF), want_r, atol=1e-5) and [n for n, _ in rms.named_parameters()] == ["weight"]
    xg, xr = x.clone().requires_grad_(), x.clone().requires_grad_()
    (ln(xg, TRAIN) * _x(4, 6, 16, seed=4)).sum().backward()
    (F.layer_norm(xr, (16,), ln.weight.tensor.detach(), ln.bias.tensor.detach(), 1e-5) * _x(4, 6, 16, seed=4)).sum().backward()
    assert torch.allclose(xg.grad, xr.grad, atol=1e-4) and ln.weight.tensor.grad is not None and ln.bias.tensor.grad is not None


# ---- dropout --------------------------------------------------------------------------------------------------------
def test_dropout_rate_scale_seed_and_gradient_mask():
    x = torch.ones(200, 200)
    d = Dropout(DropoutConfig(0.3))
    y = d(x, ForwardCtx.train(BE, seed=5))
    kept = y != 0
    assert abs(float(kept.float().mean()) - 0.7) < 0.01 and torch.allclose(y[kept], torch.full_like(y[kept], 1 / 0.7))
    assert torch.equal(d(x, ForwardCtx.train(BE, seed=5)), y) and not torch.equal(d(x, ForwardCtx.train(BE, seed=6)), y)
    ctx = ForwardCtx.train(BE, seed=5)
    first, second = d(x, ctx), d(x, ctx)
    assert torch.equal(first, y) and not torch.equal(second, first)            # each call in a context draws a fresh range
    assert d(x, INF) is x and Dropout(0.0)(x, TRAIN) is x and float(Dropout(1.0)(x, TRAIN).abs().sum()) == 0.0
    assert DropoutConfig(1.7).p == 1.0 and DropoutConfig(-0.2).p == 0.0
    xg = torch.ones(50, 50, requires_grad=True)
    yg = d(xg, ForwardCtx.train(BE, seed=9))
    yg.sum().backward()
    assert torch.equal(xg.grad != 0, yg != 0) and torch.allclose(xg.grad[xg.grad != 0], torch.tensor(1 / 0.7))


# ---- losses ---------------------------------------------------------------------------------------------------------
def test_losses_match_their_definitions_and_check_shapes():
    p, t = _x(5, 3), _x(5, 3, seed=1)
    assert float(MSELoss()(p, t)) == pytest.approx(float(((p - t) ** 2).mean()))
    with pytest.raises(ShapeMismatch):
        MSELoss()(p, t[:4])
    logits, tgt = _x(6, 4, seed=2), torch.tensor([0, 3, 1, -100, 2, -100])
    ce = CrossEntropyLoss()
    assert float(ce(logits, tgt)) == pytest.approx(float(F.cross_entropy(logits, tgt, ignore_index=-100)), abs=1e-6)
    assert float(CrossEntropyLoss(ignore_index=3)(logits, torch.tensor([0, 3, 1, 3, 2, 3]))) == pytest.approx(
        float(F.cross_entropy(logits, torch.tensor([0, 3, 1, 3, 2, 3]), ignore_index=3)), abs=1e-6)
    lg = logits.clone().requires_grad_()
    ce(lg, tgt).backward()
    lr = logits.clone().requires_grad_()
    F.cross_entropy(lr, tgt, ignore_index=-100).backward()
    assert torch.allclose(lg.grad, lr.grad, atol=1e-6) and lg.grad[3].abs().sum() == 0      # ignored rows get no gradient
    onehot = F.one_hot(torch.tensor([0, 3, 1, 2, 2, 0]), 4).float()
    assert float(ce.forward(logits, onehot)) == pytest.approx(float(F.cross_entropy(logits, onehot.argmax(-1))), abs=1e-6)
    with pytest.raises(ShapeMismatch):
        ce.forward(logits, onehot[:, :3])
    padded = torch.cat([logits, torch.full((6, 4), 50.0)], 1)                      # columns beyond n_valid must not count
    assert float(ce.forward_indices(padded, tgt, n_valid=4)) == pytest.approx(float(ce(logits, tgt)), abs=1e-6)
    x, y = _x(7, 2, seed=3) * 20, (torch.rand(7, 2, generator=torch.Generator().manual_seed(4)) > 0.5).float()
    assert float(BCEWithLogitsLoss()(x, y)) == pytest.approx(float(F.binary_cross_entropy_with_logits(x, y)), rel=1e-6)
    assert math.isfinite(float(BCEWithLogitsLoss()(torch.tensor([[1000.0, -1000.0]]), torch.tensor([[0.0, 1.0]]))))


# ---- containers -----------------------------------------------------------------------------------------------------
def test_sequential_containers_names_and_errors():
    a, b, c = (LinearBuilder(4, 4).with_bias().seed(s).build(BE) for s in (1, 2, 3))
    x = _x(2, 4)
    pair = Sequential2(a, b)
    assert torch.equal(pair(x, INF), b(a(x, INF), INF))
    assert [n for n, _ in pair.named_parameters()] == ["first.weight", "first.bias", "second.weight", "second.bias"]
    nested = chain(chain(a, b), c)
    assert [n for n, _ in nested.named_parameters()][:2] == ["first.first.weight", "first.first.bias"]
    seq = Sequential(a, b, c)
    assert torch.equal(seq(x, INF), nested(x, INF)) and seq.num_parameters() == 3 * 20
    assert torch.equal(Sequential()(x, INF), x)
    with pytest.raises(Exception):
        Sequential(a, LinearBuilder(5, 4).build(BE))(x, INF)         # 4 features into a layer that wants 5
