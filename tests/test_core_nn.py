"""Core contracts and nn modules on the CPU reference backend: naming stability, strict I/O, gradient checks, goldens."""
import json
import math
import os

import pytest
import torch

from rustral_b200.core import (CpuBackend, ForwardCtx, Mode, Shape, ShapePolicy, InvalidShape, SerializationError, ShapeMismatch,
                               OperationProfiler, MemoryProfiler, TensorPool, PoolStrategy, NumericsValidator, DType, OpFamily,
                               ToleranceConfig, FusionOptimizer, FusionPattern, PatternMatcher, FusionTestHarness, assert_close)
from rustral_b200.nn import *
from rustral_b200.optim import Adam, AdamW, Sgd, WarmupCosine, OneCycleLR, PlateauLR, StepDecay, LossScaleScheduler, MixedPrecisionOptimizer
from rustral_b200.runtime.model_io import load_model, save_model

B = CpuBackend()


def test_shape_ctx_and_capabilities():
    with pytest.raises(InvalidShape):
        Shape([])
    with pytest.raises(InvalidShape):
        Shape([3, 0])
    assert Shape([2, 3]).numel() == 6
    a, b = ForwardCtx.train(B), ForwardCtx.inference(B)
    assert a.is_training() and not b.is_training() and a.run_id != b.run_id and a.mode is Mode.TRAIN
    assert ShapePolicy.STATIC.supports_cuda_graph_capture() and not ShapePolicy.DYNAMIC_UNBOUNDED.supports_cuda_graph_capture()
    caps = B.capabilities()
    assert caps.clamp_batch_size(10_000) == caps.max_batch_size and not caps.recommends_mixed_precision()


def test_named_parameters_are_stable_and_match_the_reference_names():
    blk = TapeTransformerEncoderLayer.new(B, TapeTransformerEncoderConfig(32, 4, 64))
    names = [n for n, _ in blk.named_parameters()]
    assert names == ["ln1.weight", "ln1.bias", "attn.wq.weight", "attn.wq.bias", "attn.wk.weight", "attn.wk.bias",
                     "attn.wv.weight", "attn.wv.bias", "attn.wo.weight", "attn.wo.bias", "ln2.weight", "ln2.bias",
                     "ffn.fc1.weight", "ffn.fc1.bias", "ffn.fc2.weight", "ffn.fc2.bias"]
    enc = TransformerEncoder.new(B, TransformerEncoderConfig(32, 4, 2, 64, 0.0, 16), 50)
    n2 = [n for n, _ in enc.named_parameters()]
    assert n2[0] == "token_embedding.embed" and "layers.1.self_attn.out_proj.weight" in n2 and n2[-1] == "final_norm.bias"
    seq = chain(LinearBuilder(4, 4).build(B), LinearBuilder(4, 2).with_bias().build(B))
    assert [n for n, _ in seq.named_parameters()] == ["first.weight", "second.weight", "second.bias"]
    assert [n for n, _ in MultiHeadAttention.new(B, 32, 4).named_parameters()][0] == "attention.q_proj.weight"
    assert [n for n, _ in Embedding.new(B, 10, 4).named_parameters()] == ["embed"]


def test_every_parameter_of_a_block_gets_a_nonzero_gradient():
    ctx = ForwardCtx.train(B)
    blk = TapeTransformerEncoderLayer.new(B, TapeTransformerEncoderConfig(32, 4, 64, causal=True))
    x = torch.randn(2, 10, 32)
    blk(x, ctx).square().sum().backward()
    for n, p in blk.named_parameters():
        assert p.grad is not None and float(p.grad.abs().sum()) > 0, n


def test_linear_builder_defaults_and_fused_activations():
    a, b = LinearBuilder(6, 4).with_bias().build(B), LinearBuilder(6, 4).with_bias().build(B)
    assert torch.equal(a.weight.tensor, b.weight.tensor)                     # seed 42 by default
    assert not torch.equal(a.weight.tensor, LinearBuilder(6, 4).seed(7).build(B).weight.tensor)
    x = torch.randn(3, 6)
    g = LinearBuilder(6, 4).with_bias().activation("gelu").build(B)
    want = torch.nn.functional.gelu(x @ g.weight.tensor.t() + g.bias.tensor, approximate="tanh")
    assert torch.allclose(g(x), want, atol=1e-6)
    with pytest.raises(Exception):
        LinearBuilder(6, 4).activation("relu").build(B)                        # fused activations need a bias
    with pytest.raises(ShapeMismatch):
        a(torch.randn(3, 5))


@pytest.mark.parametrize("what", ["linear", "layer_norm", "embedding", "cross_entropy", "gelu", "rms_norm"])
def test_finite_difference_gradients(what):
    """Central differences, eps 1e-3, tolerance 1e-2 (crates/autodiff/tests/finite_difference.rs)."""
    from rustral_b200 import ops
    torch.manual_seed(0)
    if what == "linear":
        leaves = [torch.randn(3, 5), torch.randn(4, 5), torch.randn(4)]
        f = lambda x, w, b: ops.linear(x, w, b).square().sum()
    elif what == "layer_norm":
        leaves = [torch.randn(3, 8), torch.rand(8) + 0.5, torch.randn(8)]
        f = lambda x, g, b: (ops.layer_norm(x, g, b) * torch.arange(8.)).sum()
    elif what == "rms_norm":
        leaves = [torch.randn(3, 8), torch.rand(8) + 0.5]
        f = lambda x, g: (ops.rms_norm(x, g) * torch.arange(8.)).sum()
    elif what == "embedding":
        ids = torch.tensor([1, 3, 1])
        leaves = [torch.randn(5, 4)]
        f = lambda t: (ops.embedding(ids, t) * torch.arange(12.).view(3, 4)).sum()
    elif what == "cross_entropy":
        tg = torch.tensor([0, 2, 1])
        leaves = [torch.randn(3, 4)]
        f = lambda l: ops.cross_entropy(l, tg)
    else:
        leaves = [torch.randn(7)]
        f = lambda x: ops.gelu(x).sum()
    req = [l.clone().requires_grad_() for l in leaves]
    f(*req).backward()
    for li, leaf in enumerate(leaves):
        flat = leaf.reshape(-1)
        for i in range(0, flat.numel(), max(1, flat.numel() // 6)):
            def at(delta):
                mod = [l.clone() for l in leaves]
                mod[li].reshape(-1)[i] += delta
                return float(f(*mod))
            fd = (at(1e-3) - at(-1e-3)) / 2e-3
            an = float(req[li].grad.reshape(-1)[i])
            assert abs(fd - an) <= 1e-2 * max(1.0, abs(fd)), (what, li, i, fd, an)


def test_golden_softmax_against_f64():
    from rustral_b200 import ops
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0], [-1000.0, 0.0, 1000.0, 999.0]])
    want = torch.softmax(x.double(), -1)
    assert_close(ops.softmax(x), want, ToleranceConfig.for_family(OpFamily.SOFTMAX))
    assert_close(torch.exp(ops.log_softmax(x)), want, ToleranceConfig.for_family(OpFamily.SOFTMAX))


def test_model_io_roundtrip_and_strict_negatives():
    m1 = TapeTransformerEncoderLayer.new(B, TapeTransformerEncoderConfig(16, 2, 32), seed=1)
    m2 = TapeTransformerEncoderLayer.new(B, TapeTransformerEncoderConfig(16, 2, 32), seed=2)
    blob = save_model(m1)
    load_model(m2, blob)
    x = torch.randn(1, 5, 16)
    assert torch.equal(m1(x), m2(x))
    from rustral_b200.io import deserialize, serialize
    tensors, meta = deserialize(blob)
    assert "rustral.parameter_ids" in meta and set(json.loads(meta["rustral.parameter_ids"])) == set(tensors)
    for mutate in ("missing", "extra", "shape", "dtype"):
        t = dict(tensors)
        if mutate == "missing":
            t.pop("ln1.weight")
        elif mutate == "extra":
            t["bogus"] = torch.zeros(1)
        elif mutate == "shape":
            t["ln1.weight"] = torch.zeros(17)
        else:
            t["ln1.weight"] = t["ln1.weight"].to(torch.bfloat16)
        before = m2.ln1.weight.tensor.clone()
        with pytest.raises((SerializationError, ShapeMismatch)):
            load_model(m2, serialize(t))
        assert torch.equal(m2.ln1.weight.tensor, before)             # nothing was written


def test_three_runs_are_bitwise_identical():
    def run():
        torch.manual_seed(0)
        ctx = ForwardCtx.train(B)
        m = TapeTransformerEncoderLayer.new(B, TapeTransformerEncoderConfig(16, 2, 32))
        opt = Adam(1e-2)
        x = torch.randn(2, 6, 16, generator=torch.Generator().manual_seed(1))
        for _ in range(5):
            m.zero_grad()
            m(x, ctx).square().mean().backward()
            opt.step(m.parameters())
        return torch.cat([p.tensor.reshape(-1) for p in m.parameters()])
    a, b, c = run(), run(), run()
    assert torch.equal(a, b) and torch.equal(b, c)


def test_optimizers_schedulers_and_loss_scaling():
    p0 = torch.randn(50)
    g = torch.randn(50)
    from rustral_b200.core import Parameter
    for decoupled in (False, True):
        p = Parameter("p", p0.clone())
        ref = torch.nn.Parameter(p0.clone())
        ropt = (torch.optim.AdamW if decoupled else torch.optim.Adam)([ref], lr=1e-2, weight_decay=0.1, eps=1e-8)
        opt = Adam(1e-2, weight_decay=0.1, decoupled=decoupled)
        for _ in range(4):
            ref.grad = g.clone()
            ropt.step()
            opt.step([p], {p.id: g})
        assert torch.allclose(p.tensor, ref.detach(), atol=1e-6)
    p = Parameter("p", p0.clone())
    ref = torch.nn.Parameter(p0.clone())
    ropt, opt = torch.optim.SGD([ref], lr=0.1, momentum=0.9), Sgd(0.1, momentum=0.9)
    for _ in range(3):
        ref.grad = g.clone()
        ropt.step()
        opt.step([p], {p.id: g})
    assert torch.allclose(p.tensor, ref.detach(), atol=1e-6)                 # momentum is really used
    s = WarmupCosine(1e-3, 1e-5, 10, 100)
    assert s.get_lr(0) == 0 and s.get_lr(10) == pytest.approx(1e-3) and s.get_lr(100) == pytest.approx(1e-5)
    assert OneCycleLR(1.0, 100).get_lr(50) == pytest.approx(1.0) and StepDecay(1.0, 0.5, 10).get_lr(25) == 0.25
    pl = PlateauLR(1.0, 0.1, 0.5, patience=1)
    for l in (1.0, 1.0, 1.0, 1.0):
        pl.report_loss(l)
    assert pl.current_lr() == 0.5
    ls = LossScaleScheduler(1024, growth_interval=2)
    assert ls.step(True) and ls.scale == 512 and not ls.step(False) and not ls.step(False) and ls.scale == 1024
    p = Parameter("p", p0.clone())
    mp = MixedPrecisionOptimizer(Adam(1e-2), loss_scale=LossScaleScheduler(8.0))
    assert mp.step([p], {p.id: g * 8.0}) and not mp.step([p], {p.id: torch.full((50,), float("inf"))})
    q = Parameter("q", p0.clone())
    Adam(1e-2).step([q], {q.id: g})
    assert torch.allclose(p.tensor, q.tensor, atol=1e-6)                     # gradients were UNscaled before the step


def test_profilers_pool_numerics_and_fusion():
    prof = OperationProfiler(use_cuda_events=False)
    ctx = ForwardCtx.train(B, profiler=prof)
    LinearBuilder(8, 8).with_bias().build(B)(torch.randn(4, 8), ctx)
    with prof.guard("custom", (4, 8)):
        pass
    assert prof.stats["linear"].count == 1 and "4x8" in prof.stats["custom"].shape_buckets
    base = {"linear": prof.stats["linear"].mean_ms / 10}
    assert prof.check_regression(base, 0.2)[0][0] == "linear" and json.loads(prof.export_json())["linear"]["count"] == 1
    mem = MemoryProfiler(capacity_bytes=1000)
    h = mem.alloc("acts", 600)
    assert mem.predict_oom_risk(300) == "critical" and mem.find_leaks()[0][1] == "acts"
    mem.free(h)
    assert mem.current == 0 and mem.peak == 600 and len(json.loads(mem.export_timeline())) == 2
    pool = TensorPool(PoolStrategy.TRAINING_ARENA)
    t = pool.acquire((16, 16))
    pool.begin_step()
    assert pool.acquire((16, 16)) is t and pool.stats()["hits"] == 1
    v = NumericsValidator()
    assert v.validate_arrays([1.0, 2.0], [1.0, 2.0 + 1e-7]).ok and not v.validate_arrays([1.0, float("nan")], [1.0, 2.0]).ok
    assert PatternMatcher().find(["matmul", "add_row_vector", "gelu", "relu"])[0][2] is FusionPattern.MATMUL_BIAS_GELU
    x, w, b = torch.randn(5, 7), torch.randn(3, 7), torch.randn(3)
    r = FusionTestHarness(repeats=2).run_test(lambda: torch.relu(x @ w.t() + b), lambda: FusionOptimizer(B).apply_matmul_bias_relu(x, w, b))
    assert r.passed and r.max_abs_err < 1e-5


def test_onnx_export_structure_and_dashboard():
    from rustral_b200.utils import onnx_export, tui
    w, b = torch.randn(3, 4), torch.randn(3)
    blob = onnx_export.export_linear_f32(4, 3, w, b)

    def fields(buf):
        i, out = 0, []
        while i < len(buf):
            key = 0; shift = 0
            while True:
                c = buf[i]; i += 1
                key |= (c & 0x7F) << shift; shift += 7
                if not c & 0x80:
                    break
            num, wire = key >> 3, key & 7
            if wire == 0:
                v = 0; shift = 0
                while True:
                    c = buf[i]; i += 1
                    v |= (c & 0x7F) << shift; shift += 7
                    if not c & 0x80:
                        break
                out.append((num, v))
            else:
                ln = 0; shift = 0
                while True:
                    c = buf[i]; i += 1
                    ln |= (c & 0x7F) << shift; shift += 7
                    if not c & 0x80:
                        break
                out.append((num, buf[i:i + ln])); i += ln
        return out
    model = dict((n, v) for n, v in fields(blob) if n in (1, 7, 8))
    assert model[1] == 9 and dict(fields(model[8]))[2] == 17
    graph = fields(model[7])
    ops_ = [dict(fields(v))[4].decode() for n, v in graph if n == 1]
    assert ops_ == ["MatMul", "Add"]
    init = [dict(fields(v)) for n, v in graph if n == 5]
    wt = torch.frombuffer(bytearray(init[0][9]), dtype=torch.float32).view(4, 3)
    assert torch.equal(wt, w.t().contiguous())
    d = tui.TrainingDashboard()
    for i in range(5):
        tui.EpochSnapshot(i, 1.0 / (i + 1), 0.5).push_to_dashboard(d)
    import io
    assert "loss 0.2000" in tui.DashboardRenderer(d, io.StringIO(), False).render_text()


def test_gpu_profiler_chrome_trace_and_bandwidth(tmp_path):
    import json
    from rustral_b200.core.gpu_profiler import BandwidthCalculator, GpuProfiler, export_chrome_trace
    prof = GpuProfiler("cpu")
    with prof.scope("matmul", m=8):
        torch.randn(64, 64) @ torch.randn(64, 64)
    with prof.scope("copy", category="transfer"):
        torch.randn(1024).clone()
    prof.record_memory()
    trace = json.loads(export_chrome_trace(prof, str(tmp_path / "t.json")))
    names = [e["name"] for e in trace["traceEvents"]]
    assert names == ["matmul", "copy", "memory"] and trace["traceEvents"][0]["ph"] == "X"
    assert prof.summary()["matmul"]["count"] == 1
    bw = BandwidthCalculator(peak_gbs=1000.0)
    assert abs(bw.gbs(1e9, 1e6) - 1.0) < 1e-9 and abs(bw.utilization(1e9, 1e3) - 1.0) < 1e-9


def test_search_strategies_tuning_session_and_tui_hook():
    import io
    from types import SimpleNamespace
    from rustral_b200.runtime.tui_hook import TuiHook
    from rustral_b200.tune import BayesianSearch, ConfigSpace, GridSearch, TuningSession
    space = ConfigSpace({"block_n": [64, 128, 256], "group_m": [4, 8]})
    cost = lambda c: abs(c["block_n"] - 128) + c["group_m"]
    for cls in (GridSearch, BayesianSearch):
        s = cls(space, seed=1, max_evals=12)
        sess = TuningSession("gemm", "m128_n128_k128")
        while True:
            c = s.next_config()
            if c is None:
                break
            s.report(c, cost(c))
            sess.record(c, cost(c))
        sess.finish()
        best, t = s.best()
        assert best == {"block_n": 128, "group_m": 4} and t == 4
        assert sess.to_dict()["best_config"] == best
    hook = TuiHook(start_thread=False)
    hook.on_epoch(SimpleNamespace(epoch=3, train_loss=1.25))
    assert hook.dashboard.epoch == 3 and hook.dashboard.losses[-1] == 1.25
    hook.close()


def test_grad_ext_tensor_view_and_tape_trainer():
    """Gradient lookup by parameter, the zero-copy host view, and TapeTrainer end to end on a separable toy problem."""
    import numpy as np
    from rustral_b200.autograd import GradExt, Tape
    from rustral_b200.core import CpuBackend, ForwardCtx, TensorView
    from rustral_b200.core.errors import InvalidArgument
    from rustral_b200.core.module import Module, Trainable
    from rustral_b200.nn.linear import LinearBuilder
    from rustral_b200.optim import Adam
    from rustral_b200.runtime.tape_trainer import SupervisedTapeModel, Trainer
    be = CpuBackend()
    lin = LinearBuilder(3, 2).with_bias().seed(1).build(be)
    tape = Tape(ForwardCtx.train(be))
    x = tape.constant(torch.tensor([[1.0, 2.0, 3.0]]))
    w, b = tape.watch_parameter(lin.weight), tape.watch_parameter(lin.bias)
    loss = tape.sum_all_tape(tape.linear_tape(x, w, b))
    assert GradExt.gradient(lin.weight, tape) is None                       # no backward yet
    store = tape.backward(loss)
    g = GradExt.gradient(lin.weight, tape)
    assert torch.equal(g, torch.tensor([[1.0, 2.0, 3.0], [1.0, 2.0, 3.0]]))
    assert torch.equal(GradExt.gradient_from_store(lin.bias, store, tape.param_map), torch.ones(2))
    assert GradExt.gradient_from_store(lin.bias, store) is store.param_gradient(lin.bias)
    t = torch.arange(6, dtype=torch.float32).reshape(2, 3)
    v = TensorView.as_slice_f32(t)
    v[0] = 9.0
    assert isinstance(v, np.ndarray) and v.shape == (6,) and float(t[0, 0]) == 9.0      # shares memory
    with pytest.raises(InvalidArgument):
        TensorView.as_slice_f32(t.t())

    class Toy(Module, Trainable, SupervisedTapeModel):
        def __init__(self):
            self.fc = LinearBuilder(2, 2).with_bias().seed(3).build(be)

        def forward(self, x, ctx):
            return self.fc(x, ctx)

        def forward_tape(self, x, tape, ctx):
            return tape.apply("toy", lambda: self.forward(x, ctx))

    g = torch.Generator().manual_seed(0)
    xs = torch.randn(64, 2, generator=g)
    data = [(xs[i], int(xs[i, 0] > xs[i, 1])) for i in range(64)]
    rep = Trainer.classification(Adam(lr=0.1)).epochs(15).batch_size(16).seed(0).fit(be, Toy(), data)
    assert len(rep.epochs) == 15 and rep.accuracy > 0.9 and rep.epochs[-1].mean_loss < 0.5 * rep.epochs[0].mean_loss
    assert rep.throughput.examples_per_sec > 0


def test_kernel_factory_and_op_config():
    from rustral_b200.tune import (AutoTuner, ConfigCache, ConfigSpace, ConfigurableKernel, ConvAlgorithm, KernelFactory,
                                   MatmulAlgorithm, OpConfig, TunableKernel, TunerConfig)
    assert MatmulAlgorithm.TCGEN05_TWO_CTA.uses_tensor_cores() and not MatmulAlgorithm.TILED.uses_tensor_cores()
    assert MatmulAlgorithm.TENSOR_CORE_MMA.recommended_tile() == (256, 256, 64)
    a = OpConfig.matmul(MatmulAlgorithm.TILED, 128, 128, 32, 2)
    assert a == OpConfig.matmul(MatmulAlgorithm.TILED, 128, 128, 32, 2) and a != OpConfig.conv2d(ConvAlgorithm.DIRECT, 16, 64)
    assert a["block_k"] == 32 and a.to_kernel_config() == {"block_n": 128, "splits": 1, "group_m": 8}
    assert OpConfig.from_gemm_config({"block_n": 256, "splits": 1, "group_m": 8}, M=4096)["algorithm"] is MatmulAlgorithm.TCGEN05_TWO_CTA
    assert OpConfig.from_gemm_config({"block_n": 128, "splits": 4, "group_m": 8})["algorithm"] is MatmulAlgorithm.TCGEN05_SPLIT_K

    class Fake(TunableKernel, ConfigurableKernel):
        kernel_id = "fake_gemm"
        host_timed = True
        M = 4096
        calls = []

        def config_space(self):
            return ConfigSpace({"block_n": [128, 256], "splits": [1, 2], "group_m": [8]})

        def default_config(self):
            return {"block_n": 128, "splits": 2, "group_m": 8}

        def input_signature(self):
            return "m4k_n4k_k4k"

        def with_config(self, config):
            import time as _t
            cost = 0.001 if (config["block_n"], config["splits"]) == (256, 1) else 0.008
            return lambda: (Fake.calls.append(dict(config)), _t.sleep(cost))

    import tempfile
    with tempfile.TemporaryDirectory() as d:
        cfg = TunerConfig.fast()
        cfg.device_id, cfg.min_improvement_pct, cfg.warmup, cfg.timing = "test", 5.0, 1, 3
        tuner = AutoTuner(cfg, ConfigCache(os.path.join(d, "cache.json"), "test"))
        fac = KernelFactory(tuner)
        k, conf = fac.get_kernel(Fake())
        assert (conf["block_n"], conf["splits"]) == (256, 1) and tuner.stats["tuned"] == 1
        assert k.current_config()["algorithm"] is MatmulAlgorithm.TCGEN05_TWO_CTA
        n = len(Fake.calls)
        _, conf2 = fac.get_kernel(Fake())                      # second request: served from the cache, nothing timed
        assert conf2 == conf and len(Fake.calls) == n and tuner.stats["cache_hits"] == 1
        assert "matmul_default" in fac.default_configs and fac.default_configs["conv2d_default"].kind == "conv2d"


def test_check_env_reports_toolkit_libraries_and_gpus():
    from rustral_b200.utils import check_env
    assert check_env.parse_nvcc_version("Cuda compilation tools, release 12.9, V12.9.86") == (12, 9)
    assert check_env.parse_nvcc_version("garbage") is None
    info = check_env.collect()
    assert set(info["libraries"]) == {"librb200_kernels.so", "librb200_cpu.so", "librb200_runtime.so"}
    assert info["ok"] == (not info["problems"]) and isinstance(info["gpus"], list)

    class _Old:
        stdout = "release 11.8, V11.8.89"
    old = check_env.collect(run=lambda *a, **k: _Old())
    if old["nvcc"]:
        assert any("too old" in p for p in old["problems"]) and not old["ok"]


def test_gemm_tuning_table_feeds_cached_plans_back_into_gemm(tmp_path):
    """A cached winner for a shape bucket is what `ops.gemm` is asked to run with once the table is applied; explicit
    plans and uncached shapes are left alone."""
    from rustral_b200.ops import matmul
    from rustral_b200.tune import AttentionKernel, ConfigCache, GemmKernel, GemmTuningTable, MatmulShapeBucket
    cache = ConfigCache(str(tmp_path / "cache.json"), "dev0")
    key = MatmulShapeBucket.of(4096, 4096, 1024).cache_key() + "_000"
    cache.store_config(GemmKernel.kernel_id, "dev0", "bf16", key, {"block_n": 192, "splits": 2, "group_m": 8}, 10.0, 5)
    key2 = MatmulShapeBucket.of(300, 300, 300).cache_key() + "_000"
    cache.store_config(GemmKernel.kernel_id, "dev0", "bf16", key2, {"block_n": 0, "splits": 0, "group_m": 0}, 10.0, 5)
    cache.save()
    table = GemmTuningTable(ConfigCache(str(tmp_path / "cache.json"), "dev0"), device_id="dev0")
    table.cache.load()
    assert table.lookup(4096, 4096, 1024) == {"block_n": 192, "splits": 2, "group_m": 8}
    assert table.lookup(300, 300, 300) is None                 # the winner was the built-in plan
    assert table.lookup(4096, 4096, 1024, b_mn=True) is None   # another operand layout: not tuned
    assert (table.hits, table.misses) == (1, 2)
    try:
        table.apply()
        assert matmul._PLAN_HOOK == table.lookup
        x = torch.randn(8, 16)
        w = torch.randn(4, 16)
        assert torch.allclose(matmul.gemm(x, w), x @ w.t(), atol=1e-5)          # CPU tensors never consult the table
    finally:
        GemmTuningTable.remove()
    assert matmul._PLAN_HOOK is None
    k = AttentionKernel(4, 1024, 12, 12, 64)
    assert k.config_space().size() == 2 and k.default_config() == {"impl": 0}
    assert k.input_signature() == "bmedium_smedium_h12_kv12_d64_11".replace("bmedium", "btiny")
    assert k.flops() == 4.0 * 4 * 1024 * 1024 * 12 * 64 * 3.5 * 0.5


def test_safetensors_files_interoperate_with_the_reference_implementation(tmp_path):
    """Files written here are read by the `safetensors` package and the other way round: dtypes, shapes, metadata."""
    sft = pytest.importorskip("safetensors.torch")
    from rustral_b200.io import safetensors_io as st
    g = torch.Generator().manual_seed(0)
    tensors = {"w.f32": torch.randn(3, 5, generator=g), "w.bf16": torch.randn(4, 2, generator=g).bfloat16(),
               "w.f16": torch.randn(7, generator=g).half(), "ids": torch.arange(6, dtype=torch.int64).view(2, 3),
               "scalar": torch.tensor(2.5), "empty": torch.zeros(0, 4)}
    ours = str(tmp_path / "ours.safetensors")
    st.save_file(tensors, ours, {"format": "pt", "note": "written by rustral_b200"})
    theirs = sft.load_file(ours)
    assert set(theirs) == set(tensors)
    for k, v in tensors.items():
        assert theirs[k].dtype == v.dtype and theirs[k].shape == v.shape and torch.equal(theirs[k], v), k
    from safetensors import safe_open
    with safe_open(ours, framework="pt") as f:
        assert f.metadata()["note"] == "written by rustral_b200"
    other = str(tmp_path / "theirs.safetensors")
    sft.save_file({k: v.contiguous() for k, v in tensors.items()}, other, metadata={"origin": "safetensors"})
    back, meta = st.load_file(other)
    assert meta.get("origin") == "safetensors" and set(back) == set(tensors)
    for k, v in tensors.items():
        assert back[k].dtype == v.dtype and torch.equal(back[k], v), k


def test_native_token_prefetcher_serves_the_same_batches_in_order(tmp_path):
    """The C++ worker fills a ring of buffers ahead of the consumer; step for step the data equals the synchronous
    `batch(step)`, buffers are recycled only after release, and a held ring times out instead of overwriting."""
    import numpy as np
    from rustral_b200.data.datasets import TokenFileDataset
    path = tmp_path / "tokens.bin"
    np.arange(5000, dtype=np.uint16).tofile(path)
    ds = TokenFileDataset(str(path), seq_len=16, bytes_per_token=2, seed=7)
    pf = ds.prefetcher(batch_size=4, depth=3, first_step=10, pin=False)
    try:
        for s in range(10, 30):
            t, step = pf.next(timeout_s=10)
            assert step == s and torch.equal(t, ds.batch(s, 4)) and t.shape == (4, 17)
            assert bool((t[:, 1:] - t[:, :-1] == 1).all())                      # windows are contiguous runs of the file
        held = [pf.next(timeout_s=10, hold=True) for _ in range(3)]              # the whole ring in the consumer's hands
        assert [h[1] for h in held] == [30, 31, 32]
        with pytest.raises(TimeoutError):
            pf.next(timeout_s=0.2, hold=True)
        snapshot = held[0][0].clone()
        pf.release(held[1][0])
        t, step = pf.next(timeout_s=10, hold=True)
        assert step == 33 and torch.equal(held[0][0], snapshot)                  # a held buffer is never overwritten
        assert torch.equal(t, ds.batch(33, 4))
    finally:
        pf.close()
        pf.close()
    with pytest.raises(ValueError):
        TokenFileDataset(str(path), seq_len=6000, bytes_per_token=2).prefetcher(2)
    ds.close()


def test_recurrent_inference_sequences_match_the_generic_loop():
    """GruCell's one-GEMM-per-step inference path equals the differentiable per-step loop; training mode keeps gradients."""
    from rustral_b200.core import CpuBackend, ForwardCtx
    from rustral_b200.nn import GruCell, LstmCell, RnnCell
    be = CpuBackend()
    xs = torch.randn(9, 4, 12, generator=torch.Generator().manual_seed(0))
    for cls in (GruCell, LstmCell):
        cell = cls.new(be, 12, 16, seed=3)
        fast, state = cell.forward_sequence(xs, ForwardCtx.inference(be))
        slow, _ = RnnCell.forward_sequence(cell, xs, ForwardCtx.inference(be))
        assert torch.allclose(fast, slow, atol=1e-6)
        assert cls is LstmCell or not fast.requires_grad          # LstmCell's fused path is the GPU's; on the CPU it loops
        assert torch.equal(cell.hidden_of(state), fast[-1])
        train, _ = cell.forward_sequence(xs, ForwardCtx.train(be))
        assert train.requires_grad
        train.sum().backward()
        assert all(p.tensor.grad is not None for p in cell.parameters())


def test_key_padding_mask_matches_truncated_keys_and_ignores_padding_values():
    """A `KeyPaddingMask` gives every batch entry the attention over its real keys only: same result as cutting the
    padding off, whatever the padded positions hold; an entry without real keys gives zero rows."""
    from rustral_b200.nn.attention import KeyPaddingMask, scaled_dot_product_attention
    from rustral_b200.ops import attention as A
    g = torch.Generator().manual_seed(3)
    q, k, v = torch.randn(3, 6, 4, 8, generator=g), torch.randn(3, 9, 2, 8, generator=g), torch.randn(3, 9, 2, 8, generator=g)
    lens = [9, 4, 0]
    out = scaled_dot_product_attention(q, k, v, KeyPaddingMask(lens))
    for b, n in enumerate(lens):
        if n == 0:
            assert out[b].abs().max() == 0
            continue
        want = A.attention_reference(q[b:b + 1], k[b:b + 1, :n], v[b:b + 1, :n], False)
        assert torch.allclose(out[b:b + 1], want, atol=1e-6)
    k2, v2 = k.clone(), v.clone()
    k2[1, 4:], v2[1, 4:] = 1e4, -1e4                       # garbage in the padding must not leak
    assert torch.allclose(scaled_dot_product_attention(q, k2, v2, KeyPaddingMask(lens))[1], out[1], atol=1e-6)
    ids = torch.tensor([[5, 6, 7, 0, 0], [1, 0, 0, 0, 0], [1, 2, 3, 4, 5]])
    assert KeyPaddingMask.from_token_ids(ids).lengths.tolist() == [3, 1, 5]
    # gradients flow through the masked form and vanish on padded keys
    kk = k.clone().requires_grad_()
    scaled_dot_product_attention(q, kk, v, KeyPaddingMask(lens)).sum().backward()
    assert kk.grad[1, 4:].abs().max() == 0 and kk.grad[1, :4].abs().max() > 0
