"""One test per nn module, with value assertions against a plain PyTorch restatement (CPU reference backend).

Counterpart of the per-module unit tests of the reference (crates/nn/src/{normalization,quantization,lstm,moe,
expert_choice,conv,readout}.rs `mod tests`)."""
import math

import pytest
import torch

from rustral_b200.core import CpuBackend, ForwardCtx, InvalidArgument
from rustral_b200.nn import (BatchNorm, BidirectionalRnn, Conv2d, Conv2dConfig, DynamicQuantizer, ExpertChoiceConfig,
                             ExpertChoiceRouter, ExpertLayer, ExpertParallel, GPTQLinear, GruCell, LinearBuilder, LstmCell,
                             MoEConfig, MultiReadout, QATTrainer, QuantizationScheme, QuantizedLinear, QuantParams, Readout,
                             TransformerEncoderConfig, TransformerEncoderDecoder, quantize_model)

B = CpuBackend()


def _linear(i=128, o=16, seed=0):
    torch.manual_seed(seed)
    lin = LinearBuilder(i, o).with_bias().build(B)
    with torch.no_grad():
        lin.weight.tensor.copy_(torch.randn(o, i) * 0.1)
        lin.bias.tensor.copy_(torch.randn(o) * 0.1)
    return lin


# ---------------------------------------------------------------------------------------------- normalisation
def test_batch_norm_normalises_with_batch_statistics_and_tracks_running_ones():
    bn = BatchNorm.new(B, 3, eps=1e-5, momentum=0.5)
    x = torch.tensor([[1.0, 10.0, -2.0], [3.0, 30.0, -4.0], [5.0, 20.0, -6.0], [7.0, 40.0, -8.0]])
    y = bn.forward(x, ForwardCtx.train(B))
    ref = torch.nn.functional.batch_norm(x, None, None, training=True, eps=1e-5)
    assert torch.allclose(y, ref, atol=1e-6)
    assert torch.allclose(y.mean(0), torch.zeros(3), atol=1e-6) and torch.allclose(y.var(0, unbiased=False), torch.ones(3), atol=1e-4)
    # running statistics: (1 - m) * initial + m * batch
    assert torch.allclose(bn._running_mean, 0.5 * x.mean(0)) and torch.allclose(bn._running_var, 0.5 + 0.5 * x.var(0, unbiased=False))
    # inference uses them, not the batch's
    z = bn.forward(x[:1], ForwardCtx.inference(B))
    assert torch.allclose(z, (x[:1] - bn._running_mean) / torch.sqrt(bn._running_var + 1e-5), atol=1e-6)


def test_batch_norm_on_images_reduces_over_batch_and_space():
    bn = BatchNorm.new(B, 2)
    x = torch.randn(3, 2, 4, 5) * 3 + 1
    y = bn.forward(x, ForwardCtx.train(B))
    assert torch.allclose(y, torch.nn.functional.batch_norm(x, None, None, training=True), atol=1e-5)


# ---------------------------------------------------------------------------------------------- quantisation
def test_quant_params_round_trip_error_is_at_most_half_a_step():
    t = torch.linspace(-3, 5, 1001)
    for symmetric in (True, False):
        p = QuantParams.from_tensor(t, symmetric=symmetric)
        err = (p.dequantize(p.quantize(t)) - t).abs().max()
        assert float(err) <= 0.5 * float(p.scale) + 1e-6
    assert float(QuantParams.from_tensor(t, symmetric=False).scale) < float(QuantParams.from_tensor(t, symmetric=True).scale)
    assert DynamicQuantizer().roundtrip_error(t) <= 0.5 * 5 / 127 + 1e-6


@pytest.mark.parametrize("scheme,bound", [(QuantizationScheme.INT8, 0.02), (QuantizationScheme.INT8_ASYMMETRIC, 0.02),
                                          (QuantizationScheme.INT8_PER_CHANNEL, 0.015), (QuantizationScheme.FP8_E4M3, 0.08),
                                          (QuantizationScheme.FP8_E5M2, 0.15)])
def test_quantized_linear_stays_close_to_the_dense_layer(scheme, bound):
    lin = _linear()
    x = torch.randn(6, 128)
    q = QuantizedLinear.from_linear(lin, scheme)
    ref = lin(x)
    rel = float((q(x) - ref).norm() / ref.norm())
    assert rel < bound, rel
    assert q.qweight.element_size() == 1 and q.memory_bytes() < lin.weight.tensor.numel() * 4 / 3.5
    # the stored weight dequantises to within one quantisation step per element
    step = 0.07 if scheme is QuantizationScheme.FP8_E4M3 else 0.14 if scheme is QuantizationScheme.FP8_E5M2 else 0.01
    assert float((q.dequantized_weight() - lin.weight.tensor).abs().max() / lin.weight.tensor.abs().max()) < step


def test_fp8_linear_equals_its_definition():
    """e4m3 weights with per-channel scales, tokens quantised per row: the layer's output is exactly the product of the
    dequantised operands (fp32 accumulation) plus the bias."""
    from rustral_b200.ops import quant as Q
    lin = _linear(64, 8, seed=3)
    q = QuantizedLinear.from_linear(lin, QuantizationScheme.FP8_E4M3)
    x = torch.randn(5, 64)
    a8, sa = Q.quantize_fp8_rows(x)
    assert a8.dtype == torch.uint8 and torch.allclose(sa, x.abs().amax(1) / 448.0)
    xa = a8.view(torch.float8_e4m3fn).float() * sa[:, None]
    assert float((xa - x).abs().max()) <= float(x.abs().max()) * 2 ** -4          # three mantissa bits
    want = xa @ q.dequantized_weight().t() + lin.bias.tensor
    assert torch.allclose(q(x), want, atol=1e-5, rtol=1e-5)
    zeros, sz = Q.quantize_fp8_rows(torch.zeros(2, 32))
    assert not zeros.any() and torch.equal(sz, torch.ones(2))


def test_gptq_linear_packs_two_nibbles_per_byte_and_bounds_the_group_error():
    lin = _linear(128, 16, seed=1)
    g = GPTQLinear.from_linear(lin, 64)
    assert g.packed.shape == (16, 64) and g.packed.dtype == torch.uint8 and g.scales.shape == (16, 2)
    w, wq = lin.weight.tensor, g.dequantized_weight()
    # every element is within half a step of its group's grid
    step = g.scales.repeat_interleave(64, 1)
    assert bool(((wq - w).abs() <= 0.5 * step + 1e-6).all())
    x = torch.randn(4, 128)
    ref = lin(x)
    assert float((g(x) - ref).norm() / ref.norm()) < 0.12
    assert g.memory_bytes() < w.numel() * 4 / 6
    from rustral_b200.ops import quant as Q
    assert torch.equal(Q.dequant_int4(g.packed, g.scales, 64).float(), wq.to(torch.bfloat16).float())
    with pytest.raises(InvalidArgument):
        GPTQLinear.from_linear(_linear(100, 4), 64)


def test_fake_quantisation_passes_gradients_straight_through():
    t = torch.linspace(-1, 1, 41, requires_grad=True)
    fq = QATTrainer.fake_quantize(t, 4)
    levels = torch.unique(fq.detach())
    assert len(levels) <= 16 and float((fq - t).abs().max()) <= 0.5 / 7 + 1e-6
    (fq * torch.arange(41.0)).sum().backward()
    assert torch.equal(t.grad, torch.arange(41.0))


def test_quantize_model_replaces_every_linear():
    class Two:
        def __init__(self):
            self.a, self.b, self.rest = _linear(64, 8), [_linear(64, 8, 1), _linear(64, 8, 2)], 3

        def named_parameters(self):
            return []
    m = Two()
    assert quantize_model(m, QuantizationScheme.INT4, 32) == 3 and isinstance(m.a, GPTQLinear) and isinstance(m.b[1], GPTQLinear)
    m2 = Two()
    assert quantize_model(m2, QuantizationScheme.FP8_E4M3) == 3 and m2.b[0].is_fp8


# ---------------------------------------------------------------------------------------------- recurrent
def test_lstm_cell_matches_torch_lstm_cell():
    """Gate order here is input, forget, output, cell; torch's is input, forget, cell, output."""
    I, H = 6, 5
    cell = LstmCell.new(B, I, H)
    with torch.no_grad():
        cell.b.tensor.copy_(torch.randn(4 * H) * 0.1)
    ref = torch.nn.LSTMCell(I, H)
    order = torch.cat([torch.arange(0, 2 * H), torch.arange(3 * H, 4 * H), torch.arange(2 * H, 3 * H)])   # i f g o <- i f o g
    with torch.no_grad():
        ref.weight_ih.copy_(cell.wx.tensor[order]); ref.weight_hh.copy_(cell.wh.tensor[order])
        ref.bias_ih.copy_(cell.b.tensor[order]); ref.bias_hh.zero_()
    xs = torch.randn(4, 3, I)
    out, (h, c) = cell.forward_sequence(xs, ForwardCtx.inference(B))
    hr, cr = torch.zeros(3, H), torch.zeros(3, H)
    for t in range(4):
        hr, cr = ref(xs[t], (hr, cr))
        assert torch.allclose(out[t], hr, atol=1e-6)
    assert torch.allclose(h, hr, atol=1e-6) and torch.allclose(c, cr, atol=1e-6)


def test_bidirectional_rnn_concatenates_forward_and_reversed_backward_passes():
    f, b = GruCell.new(B, 4, 3, seed=1), GruCell.new(B, 4, 3, seed=2)
    bi = BidirectionalRnn(f, b)
    xs = torch.randn(5, 2, 4)
    ctx = ForwardCtx.inference(B)
    out, _ = bi.forward_sequence(xs, ctx)
    of, _ = f.forward_sequence(xs, ctx)
    ob, _ = b.forward_sequence(torch.flip(xs, (0,)), ctx)
    assert out.shape == (5, 2, 6)
    assert torch.equal(out[..., :3], of) and torch.equal(out[..., 3:], torch.flip(ob, (0,)))
    # the backward half at time 0 has seen the whole sequence, the forward half only the first element
    xs2 = xs.clone(); xs2[-1] += 1.0
    out2, _ = bi.forward_sequence(xs2, ctx)
    assert torch.equal(out2[0, :, :3], out[0, :, :3]) and not torch.equal(out2[0, :, 3:], out[0, :, 3:])
    assert bi.final_hidden(xs, ctx).shape == (2, 6)


# ---------------------------------------------------------------------------------------------- transformer
def test_encoder_decoder_is_causal_in_the_target_and_sees_the_whole_source():
    cfg = TransformerEncoderConfig(32, 4, 1, 64, 0.0, 16)
    m = TransformerEncoderDecoder.new(B, cfg, 20, 30)
    ctx = ForwardCtx.inference(B)
    src = torch.tensor([[1, 2, 3, 4, 5]]); tgt = torch.tensor([[7, 8, 9, 10]])
    y = m.forward((src, tgt), ctx)
    assert y.shape[:2] == (1, 4) and y.shape[-1] == 30
    tgt2 = tgt.clone(); tgt2[0, 3] = 11
    y2 = m.forward((src, tgt2), ctx)
    assert torch.allclose(y[:, :3], y2[:, :3], atol=1e-6) and not torch.allclose(y[:, 3], y2[:, 3])
    src2 = src.clone(); src2[0, 4] = 9
    y3 = m.forward((src2, tgt), ctx)
    assert not torch.allclose(y[:, 0], y3[:, 0])
    out = m.generate(src, ctx, bos=1, eos=2, max_len=5)
    assert out[0] == 1 and 2 <= len(out) <= 6 and all(0 <= t < 30 for t in out)


# ---------------------------------------------------------------------------------------------- mixture of experts
def test_expert_layer_balances_and_trains_every_parameter():
    ctx = ForwardCtx.train(B)
    layer = ExpertLayer.new(B, MoEConfig(32, 4, 64, 2))
    x = torch.randn(3, 10, 32, requires_grad=True)
    out = layer(x, ctx)
    (out.output.sum() + out.aux_loss).backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in layer.parameters())
    assert out.output.shape == x.shape and 0 < float(out.aux_loss.detach()) < 0.1
    assert ExpertParallel(8, 4, 1).local_experts() == [1, 5]


def test_expert_choice_gives_every_expert_its_capacity_and_reports_unrouted_tokens():
    cfg = ExpertChoiceConfig(8, 3, 16, tokens_per_expert=2)
    r = ExpertChoiceRouter.new(B, cfg)
    with torch.no_grad():
        r.router.tensor.zero_()
        r.router.tensor[0, 0] = 5.0; r.router.tensor[1, 1] = 5.0; r.router.tensor[2, 2] = 5.0
    x = torch.zeros(6, 8)
    x[0, 0] = 2.0; x[1, 0] = 1.0; x[2, 1] = 2.0; x[3, 1] = 1.0; x[4, 2] = 2.0; x[5, 2] = 1.0
    idx, gate, probs = r.select(x)
    assert [sorted(row.tolist()) for row in idx] == [[0, 1], [2, 3], [4, 5]]
    assert torch.allclose(probs.sum(-1), torch.ones(6), atol=1e-6) and torch.allclose(gate, probs.t().gather(1, idx))
    y = r.forward(x, lambda e, rows: rows * (e + 1), ForwardCtx.inference(B))
    want = torch.zeros_like(x)
    for e in range(3):
        for t_i, g in zip(idx[e].tolist(), gate[e].tolist()):
            want[t_i] += g * x[t_i] * (e + 1)
    assert torch.allclose(y, want, atol=1e-6)
    st = r.last_stats
    assert (st.min_tokens, st.max_tokens, st.avg_tokens, st.imbalance, st.unrouted_tokens) == (2, 2, 2.0, 1.0, 0)
    # with capacity 1 only three of the six tokens are served
    r1 = ExpertChoiceRouter.new(B, ExpertChoiceConfig(8, 3, 16, tokens_per_expert=1))
    r1.router.tensor.data.copy_(r.router.tensor)
    r1.forward(x, lambda e, rows: rows, ForwardCtx.inference(B))
    assert r1.last_stats.unrouted_tokens == 3
    with pytest.raises(InvalidArgument):
        ExpertChoiceRouter.new(B, ExpertChoiceConfig(8, 3, 16, tokens_per_expert=9)).forward(x, lambda e, rows: rows, ForwardCtx.inference(B))


# ---------------------------------------------------------------------------------------------- conv, readouts
def test_conv2d_matches_torch_conv2d_forward_and_gradients():
    conv = Conv2d.new(B, Conv2dConfig(5, 3, 3, in_channels=2))
    img = torch.randn(2, 2, 8, 8, requires_grad=True)
    y = conv(img)
    ref_in = img.detach().clone().requires_grad_()
    ref = torch.nn.functional.conv2d(ref_in, conv.weight.tensor, conv.bias.tensor, padding=1)
    assert torch.allclose(y, ref, atol=1e-5)
    y.square().sum().backward(); ref.square().sum().backward()
    assert torch.allclose(img.grad, ref_in.grad, atol=1e-4)


def test_readouts_return_labels_with_probabilities():
    from rustral_b200.symbolic import Vocabulary
    ctx = ForwardCtx.inference(B)
    labels = Vocabulary.with_specials("<unk>", ["pos", "neg"])
    ro = Readout.new(B, labels, 8)
    h = torch.randn(3, 8)
    pred = ro.predict(h, ctx)
    assert len(pred) == 3 and all(p.label in labels.tokens() and 0 <= p.score <= 1 for p in pred)
    top = MultiReadout.new(B, ["a", "b", "c"], 8).top_k(h[:2], ctx, 2)
    assert len(top) == 2 and len(top[0]) == 2 and top[0][0].score >= top[0][1].score


# ---------------------------------------------------------------------------------------------- dashboard
def test_dashboard_panes_keys_leak_warnings_and_json_dump(tmp_path):
    import io
    import json
    import time
    from rustral_b200.core import MemoryProfiler
    from rustral_b200.utils import tui
    cfg = tui.DashboardConfig(title="run-7", history_len=16, dump_path=str(tmp_path / "state.json"), alt_screen=False)
    d = tui.TrainingDashboard(config=cfg)
    d.set_total_epochs(4); d.set_total_batches(10); d.set_epoch(1); d.set_batch(5); d.set_step(15)
    for i in range(40):
        d.record_loss(2.0 / (i + 1)); d.record_lr(1e-3 * 0.9 ** i)
    d.record_accuracy(0.75)
    assert len(d.losses) == 16 and d.current_loss() == 2.0 / 40          # rolling window
    d.record_loss(float("nan"))
    assert any("non-finite loss" in w for w in d.warnings)
    prof = MemoryProfiler(capacity_bytes=1000)
    prof.alloc("weights", 600); h = prof.alloc("activations", 320); prof.free(h); prof.alloc("scratch", 330)
    d.attach_memory_profiler(prof, leak_age_s=0.0)
    keys = iter(["", "p", "p", "c", "zq"])
    r = tui.DashboardRenderer(d, io.StringIO(), ansi=False, width=90, keys=lambda: next(keys))
    assert r.render_frame() is False
    assert d.oom_risk_level() is tui.OomRiskLevel.CRITICAL and d.memory_used == 930 and d.memory_peak == 930
    assert sorted(l.tag for l in d.leaks) == ["scratch", "weights"] and (d.allocs, d.deallocs) == (3, 1)
    panes = r.render_panes(90)
    for needle in ("┌─ progress", "┌─ metrics", "┌─ memory", "┌─ warnings and events", "epoch     1/4", "batch     5/10",
                   "OOM risk: CRITICAL", "LEAK weights: 600 B", "weights", "q quit"):
        assert needle in panes, needle
    assert all(len(line) == 90 for line in panes.splitlines()[1:])            # every box line fills the width
    state = json.loads((tmp_path / "state.json").read_text())
    assert state["memory"]["oom_risk"] == "critical" and len(state["leaks"]) == 2 and state["step"] == 15
    assert r.render_frame() is False and r.paused                           # "p"
    assert r.render_frame() is False and not r.paused                       # "p" again
    assert r.render_frame() is False and d.has_leaks()                      # "c" clears; the same frame's poll finds them again
    assert r.handle_key("c") is False and not d.has_leaks()
    assert r.render_frame() is True and not r.is_running()                  # unknown key ignored, then "q"
    # a config handed to run_dashboard yields a dashboard with a render thread that stops on request
    d2 = tui.run_dashboard(tui.DashboardConfig(refresh_ms=10, alt_screen=False), file=io.StringIO())
    d2.record_loss(1.0)
    time.sleep(0.05)
    d2.render_thread.stop_event.set()
    d2.render_thread.join(timeout=2)
    assert not d2.render_thread.is_alive()
    assert tui.format_bytes(1536) == "1.50 KiB" and tui.format_duration(3725) == "1:02:05" and tui.format_duration(None) == "--:--"
