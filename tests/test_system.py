"""System-level checks on the CPU reference backend, after the reference's system suite (tests/edge_cases/mod.rs,
tests/bug_regression/mod.rs, tests/stress/mod.rs): degenerate shapes, extreme and special values, error paths that
must raise instead of corrupting state, determinism, and sustained use without growth."""
import gc
import math
import threading

import pytest
import torch

from rustral_b200 import ops
from rustral_b200.core import CpuBackend, ForwardCtx
from rustral_b200.core.errors import InvalidArgument, ShapeMismatch
from rustral_b200.nn import Dropout, Embedding, LayerNorm, LinearBuilder, TransformerEncoder, TransformerEncoderConfig
from rustral_b200.nn.attention import causal_mask, scaled_dot_product_attention
from rustral_b200.optim import Adam
from rustral_b200.runtime.model_io import load_model, save_model

BE = CpuBackend()
T = BE.ops()


# ---- edge cases -----------------------------------------------------------------------------------------------------
def test_single_element_wide_and_narrow_tensors():
    one = T.tensor_from_vec([3.0], (1, 1))
    assert T.tensor_to_vec(T.matmul(one, one)) == [9.0] and T.tensor_to_vec(T.softmax(one)) == [1.0]
    wide, narrow = torch.ones(1, 4096), torch.ones(4096, 1)
    assert float(T.matmul(wide, narrow)) == 4096.0 and T.matmul(narrow, wide).shape == (4096, 4096)
    assert torch.allclose(T.softmax(wide), torch.full((1, 4096), 1 / 4096))
    lin = LinearBuilder(1, 1).with_bias().build(BE)
    assert lin(torch.ones(1, 1)).shape == (1, 1)


def test_zero_sized_and_mismatched_shapes_raise_or_stay_empty():
    with pytest.raises((ShapeMismatch, InvalidArgument, ValueError)):
        T.matmul(torch.ones(2, 3), torch.ones(4, 2))
    with pytest.raises((ShapeMismatch, InvalidArgument, ValueError)):
        T.tensor_from_vec([1.0, 2.0, 3.0], (2, 2))
    with pytest.raises((ShapeMismatch, InvalidArgument, ValueError, RuntimeError)):
        LinearBuilder(4, 2).build(BE)(torch.ones(3, 5))
    with pytest.raises((ShapeMismatch, InvalidArgument, ValueError)):
        T.reshape(torch.ones(2, 3), (4, 2))
    emb = Embedding.new(BE, 10, 4)
    with pytest.raises(InvalidArgument):
        emb([10])
    with pytest.raises(InvalidArgument):
        emb([-1])
    assert T.zeros((0, 4)).numel() == 0 and T.concat([torch.ones(0, 3), torch.ones(2, 3)], 0).shape == (2, 3)


def test_extreme_and_special_values():
    big = torch.tensor([[1e30, -1e30, 0.0], [88.0, 89.0, 90.0]])
    sm = T.softmax_dim(big, -1)
    assert torch.isfinite(sm).all() and torch.allclose(sm.sum(-1), torch.ones(2))          # max-subtracted: no overflow
    assert torch.allclose(sm[0], torch.tensor([1.0, 0.0, 0.0]))
    ls = T.log_softmax_dim(big, -1)
    assert torch.isfinite(ls[1]).all() and ls[0, 0] == 0.0
    x = torch.tensor([[float("nan"), 1.0], [float("inf"), -float("inf")]])
    assert torch.isnan(T.add(x, x)[0, 0]) and T.relu(x)[1, 0] == float("inf") and T.relu(x)[1, 1] == 0.0
    assert math.isnan(float(T.sum_all(x)))                                                   # NaN propagates, never hidden
    tiny = torch.full((4, 8), 1e-30)
    ln = LayerNorm.new(BE, 8)
    assert torch.isfinite(ln(tiny)).all()                                                    # eps keeps the division finite
    logits = torch.tensor([[1e4, -1e4, 0.0]])
    assert float(ops.cross_entropy(logits, torch.tensor([0]))) == pytest.approx(0.0, abs=1e-6)
    assert float(ops.cross_entropy(logits, torch.tensor([1]))) == pytest.approx(2e4, rel=1e-6)


def test_division_log_and_sqrt_domain_errors_are_reported():
    with pytest.raises((InvalidArgument, ZeroDivisionError, ValueError)):
        T.div(torch.ones(3), torch.tensor([1.0, 0.0, 2.0]))
    with pytest.raises((InvalidArgument, ValueError)):
        T.log(torch.tensor([1.0, -1.0]))
    with pytest.raises((InvalidArgument, ValueError)):
        T.sqrt(torch.tensor([4.0, -4.0]))
    assert torch.allclose(T.div(torch.ones(2), torch.tensor([2.0, 4.0])), torch.tensor([0.5, 0.25]))


def test_causal_mask_boundaries_and_sequence_lengths():
    for S in (1, 2, 17):
        m = causal_mask(BE, S)
        assert m.shape == (S, S) and (m.diagonal() == 0).all() and (torch.tril(m) == 0).all()
        if S > 1:
            assert m[0, 1] == float("-inf") and m[S - 1, 0] == 0
    q = k = v = torch.randn(1, 5, 2, 8, generator=torch.Generator().manual_seed(0))
    o = scaled_dot_product_attention(q, k, v, None, True)
    assert torch.allclose(o[:, 0], v[:, 0], atol=1e-6)                                       # the first token sees only itself
    v2 = v.clone()
    v2[:, 4] += 100.0
    o2 = scaled_dot_product_attention(q, k, v2, None, True)
    assert torch.allclose(o[:, :4], o2[:, :4], atol=1e-6)                                    # the future never leaks back
    cfg = TransformerEncoderConfig(16, 2, 1, 32, dropout=0.0, max_seq_len=8, vocab_size=11)
    enc = TransformerEncoder.new(BE, cfg)
    assert enc.forward([[1, 2, 3, 4, 5, 6, 7, 8]], ForwardCtx.inference(BE)).shape == (1, 8, 16)
    with pytest.raises(InvalidArgument):
        enc.forward([list(range(9))], ForwardCtx.inference(BE))                             # one past max_seq_len


def test_non_contiguous_inputs_give_the_same_result():
    g = torch.Generator().manual_seed(1)
    a, b = torch.randn(6, 8, generator=g), torch.randn(8, 5, generator=g)
    at = a.t().contiguous().t()                                                              # same values, column-major strides
    assert not at.is_contiguous() and torch.allclose(T.matmul(at, b), T.matmul(a, b), atol=1e-6)
    x = torch.randn(4, 10, generator=g)[:, ::2]
    assert torch.allclose(T.softmax_dim(x, -1), torch.softmax(x.contiguous(), -1), atol=1e-6)
    assert torch.allclose(T.softmax(x).sum(), torch.tensor(1.0), atol=1e-6)                  # `softmax` is over ALL elements
    lin = LinearBuilder(5, 3).with_bias().build(BE)
    assert torch.allclose(lin(x), lin(x.contiguous()), atol=1e-6)


# ---- regressions ----------------------------------------------------------------------------------------------------
def test_dropout_is_mode_gated_seeded_and_unbiased():
    x = torch.ones(200, 50)
    d = Dropout(0.3)
    assert torch.equal(d(x, ForwardCtx.inference(BE)), x)                                     # inference: identity
    a, b = T.dropout_with_seed(x, 0.3, 7), T.dropout_with_seed(x, 0.3, 7)
    c = T.dropout_with_seed(x, 0.3, 8)
    assert torch.equal(a, b) and not torch.equal(a, c)
    kept = (a != 0).float().mean().item()
    assert abs(kept - 0.7) < 0.02 and a.max().item() == pytest.approx(1 / 0.7)               # inverted scaling
    assert abs(a.mean().item() - 1.0) < 0.03
    with pytest.raises((InvalidArgument, ValueError)):
        T.dropout_with_seed(x, 1.5, 0)


def test_gradient_overflow_is_visible_and_clipped_updates_stay_finite():
    lin = LinearBuilder(4, 2).with_bias().seed(2).build(BE)
    x = torch.full((2, 4), 1e20)
    loss = lin(x, ForwardCtx.train(BE)).pow(2).sum()
    loss.backward()
    g = lin.weight.tensor.grad
    assert not torch.isfinite(g).all()                                                       # overflow is not masked ...
    before = lin.weight.tensor.detach().clone()
    torch.nn.utils.clip_grad_norm_([lin.weight.tensor, lin.bias.tensor], 1.0, error_if_nonfinite=False)
    lin.weight.tensor.grad = torch.nan_to_num(lin.weight.tensor.grad, nan=0.0, posinf=0.0, neginf=0.0)
    lin.bias.tensor.grad = torch.nan_to_num(lin.bias.tensor.grad, nan=0.0, posinf=0.0, neginf=0.0)
    Adam(lr=1e-3).step(lin.parameters())
    assert torch.isfinite(lin.weight.tensor).all() and (lin.weight.tensor - before).abs().max() <= 2e-3


def test_save_load_consistency_and_strict_negatives():
    from rustral_b200.core.errors import SerializationError
    a = LinearBuilder(6, 3).with_bias().seed(1).build(BE)
    b = LinearBuilder(6, 3).with_bias().seed(99).build(BE)
    x = torch.randn(5, 6, generator=torch.Generator().manual_seed(3))
    assert not torch.equal(a(x), b(x))
    blob = save_model(a)
    for _ in range(3):                                                                       # repeated serialisation is stable
        assert save_model(a) == blob
    load_model(b, blob)
    assert torch.equal(a(x), b(x))
    wrong = LinearBuilder(6, 4).with_bias().build(BE)
    with pytest.raises((ShapeMismatch, SerializationError)):
        load_model(wrong, blob)
    nobias = LinearBuilder(6, 3).build(BE)
    with pytest.raises(SerializationError):
        load_model(nobias, blob)                                                             # extra key
    with pytest.raises(SerializationError):
        load_model(a, save_model(nobias))                                                    # missing key
    with pytest.raises(SerializationError):
        load_model(a, blob[: len(blob) // 2])                                                # truncated file


def test_quantization_error_is_bounded():
    q = BE.quantization_ops()
    w = torch.randn(64, 64, generator=torch.Generator().manual_seed(5))
    qi, scale = q.quantize_int8(w)
    back = q.dequantize_int8(qi, scale)
    assert qi.dtype == torch.int8 and (back - w).abs().max() <= scale * 0.5 + 1e-6           # at most half a step


# ---- stress ---------------------------------------------------------------------------------------------------------
def test_sustained_forward_and_allocation_churn_do_not_grow():
    cfg = TransformerEncoderConfig(32, 4, 2, 64, dropout=0.0, max_seq_len=16, vocab_size=50)
    enc = TransformerEncoder.new(BE, cfg)
    ctx = ForwardCtx.inference(BE)
    ids = [[(i * 7 + j) % 50 for j in range(16)] for i in range(4)]
    first = enc.forward(ids, ctx)
    gc.collect()
    base = len(gc.get_objects())
    for _ in range(60):
        out = enc.forward(ids, ctx)
        tmp = [T.zeros((64, 64)) for _ in range(20)]
        del tmp
    gc.collect()
    assert torch.equal(out, first)                                                           # same input, same output, every time
    assert len(gc.get_objects()) - base < 2000                                               # no per-call object leak


def test_concurrent_model_usage_and_error_recovery():
    lin = LinearBuilder(16, 16).with_bias().seed(4).build(BE)
    x = torch.randn(8, 16, generator=torch.Generator().manual_seed(6))
    want = lin(x)
    results, errors = [None] * 8, []

    def worker(i):
        try:
            for _ in range(50):
                y = lin(x)
            results[i] = y
        except Exception as e:      # noqa: BLE001
            errors.append(e)
    threads = [threading.Thread(target=worker, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=60)
    assert not errors and all(torch.equal(r, want) for r in results)
    for _ in range(20):                                                                      # failures leave the layer usable
        with pytest.raises((ShapeMismatch, InvalidArgument, ValueError, RuntimeError)):
            lin(torch.ones(3, 5))
        assert torch.equal(lin(x), want)


def test_gradient_accumulation_over_many_micro_batches_matches_one_batch():
    lin = LinearBuilder(8, 4).with_bias().seed(7).build(BE)
    g = torch.Generator().manual_seed(8)
    x, y = torch.randn(64, 8, generator=g), torch.randn(64, 4, generator=g)
    ctx = ForwardCtx.train(BE)
    ((lin(x, ctx) - y).pow(2).mean()).backward()
    full = lin.weight.tensor.grad.clone()
    lin.zero_grad()
    for i in range(0, 64, 4):
        ((lin(x[i:i + 4], ctx) - y[i:i + 4]).pow(2).mean() / 16).backward()
    assert torch.allclose(lin.weight.tensor.grad, full, atol=1e-6)


def test_long_sequence_attention_matches_blockwise_evaluation():
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn(1, 2048, 2, 16, generator=g) for _ in range(3))
    o = scaled_dot_product_attention(q, k, v, None, True)
    assert torch.isfinite(o).all()
    tail = scaled_dot_product_attention(q[:, -64:], k, v, None, False)                       # last rows see everything
    assert torch.allclose(o[:, -1], tail[:, -1], atol=1e-5)
