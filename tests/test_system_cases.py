"""System suite: the bug-regression, edge-case and stress cases of the reference that `tests/test_system.py` does not
already hold as a test of their own (tests/bug_regression/mod.rs, tests/edge_cases/mod.rs, tests/stress/mod.rs), plus its
performance category (tests/performance/mod.rs) as timed runs with sanity bounds.  CPU reference backend."""
import gc
import math
import threading
import time

import pytest
import torch

from rustral_b200 import ops
from rustral_b200.core import CpuBackend, ForwardCtx, MemoryProfiler, TensorPool
from rustral_b200.core.errors import InvalidArgument, InvalidShape, ShapeMismatch
from rustral_b200.nn import (Conv2d, Conv2dConfig, Embedding, LayerNorm, LinearBuilder, Sequential, TransformerDecoder,
                             TransformerDecoderConfig, TransformerEncoder, TransformerEncoderConfig)
from rustral_b200.nn.attention import scaled_dot_product_attention
from rustral_b200.optim import Adam
from rustral_b200.runtime.model_io import load_model, save_model

BE = CpuBackend()
T = BE.ops()
ERRORS = (ShapeMismatch, InvalidShape, InvalidArgument, ValueError, RuntimeError, IndexError)


# ---- bug regression -------------------------------------------------------------------------------------------------
def test_empty_input_is_rejected_or_stays_empty():
    lin = LinearBuilder(4, 2).with_bias().build(BE)
    out = lin(torch.zeros(0, 4))
    assert out.shape == (0, 2)
    assert T.tensor_from_vec([], (0,)).numel() == 0 and T.tensor_to_vec(T.zeros((0, 3))) == []
    enc = TransformerEncoder.new(BE, TransformerEncoderConfig(16, 2, 1, 32, 0.0, 8), 20)
    try:
        y = enc.forward([[]], ForwardCtx.inference(BE))        # an empty sequence: refused, or an empty result
        assert y.numel() == 0
    except ERRORS:
        pass


def test_large_tensor_allocation_and_release():
    t = T.zeros((4096, 4096))                       # 64 MiB
    assert t.shape == (4096, 4096) and float(t.sum()) == 0.0
    del t
    gc.collect()
    prof = MemoryProfiler(capacity_bytes=1 << 30)
    h = prof.alloc("big", 900 << 20)
    assert prof.predict_oom_risk(200 << 20) in ("high", "critical", "HIGH", "CRITICAL") or "high" in str(prof.predict_oom_risk(200 << 20)).lower() \
        or "crit" in str(prof.predict_oom_risk(200 << 20)).lower()
    prof.free(h)
    assert prof.current == 0 and prof.peak == 900 << 20


def test_incompatible_dimensions_raise_and_name_the_shapes():
    with pytest.raises(ERRORS) as e:
        T.matmul(torch.ones(2, 3), torch.ones(4, 5))
    assert "3" in str(e.value) or "4" in str(e.value)
    with pytest.raises(ERRORS):
        T.add(torch.ones(2, 3), torch.ones(3, 2))
    with pytest.raises(ERRORS):
        LinearBuilder(8, 2).build(BE)(torch.ones(4, 7))


def test_layers_do_not_leak_tracked_memory():
    prof = MemoryProfiler(capacity_bytes=1 << 30)
    lin = LinearBuilder(32, 32).build(BE)
    for i in range(50):
        with prof.track_tensor(f"act{i}", lin(torch.ones(8, 32))):
            pass
    assert prof.find_leaks() == [] and prof.current == 0
    held = prof.track_tensor("held", torch.ones(16))
    assert [tag for _, tag, _ in prof.find_leaks()] == ["held"]
    held.release()
    assert prof.find_leaks() == []


def test_batch_size_mismatch_between_inputs_and_targets():
    from rustral_b200.nn import CrossEntropyLoss, MSELoss
    with pytest.raises(ERRORS):
        CrossEntropyLoss()(torch.randn(4, 3), torch.tensor([0, 1, 2]))
    with pytest.raises(ERRORS):
        MSELoss()(torch.randn(4, 3), torch.randn(5, 3))


def test_nan_propagates_and_is_detectable():
    lin = LinearBuilder(4, 4).with_bias().build(BE)
    x = torch.ones(2, 4)
    x[0, 1] = float("nan")
    y = lin(x)
    assert torch.isnan(y[0]).all() and not torch.isnan(y[1]).any()      # only the poisoned row
    from rustral_b200.core import NumericsValidator
    assert not NumericsValidator().validate_arrays(y.detach().flatten().tolist(), [0.0] * 8).ok


def test_concurrent_access_to_shared_state_is_consistent():
    pool = TensorPool()
    errors = []

    def worker():
        try:
            for _ in range(200):
                t = pool.acquire((32, 32))
                t.fill_(1.0)
                pool.release(t)
        except Exception as e:          # noqa: BLE001
            errors.append(e)
    ths = [threading.Thread(target=worker) for _ in range(8)]
    for t in ths:
        t.start()
    for t in ths:
        t.join(timeout=60)
    st = pool.stats()
    assert not errors and st["hits"] + st["misses"] == 1600


def test_resource_exhaustion_is_an_error_not_a_crash():
    from rustral_b200.serve.kv_cache import PagedCache
    cache = PagedCache(4, 16, 1, 1, 8, torch.float32, "cpu")
    assert cache.allocate(1, 64) and not cache.allocate(2, 16)           # all four blocks taken
    cache.free(1)
    assert cache.allocate(2, 16) and cache.free_blocks == 3


def test_runaway_loops_are_bounded():
    """Generation stops at max_tokens even when the model never emits the end token; a step watchdog reports a stall."""
    from rustral_b200.models.config import preset
    from rustral_b200.serve.engine import ServingEngine
    from rustral_b200.serve.model_runner import ModelRunner
    cfg = preset("gpt2-test", seq_len=32, d_model=32, ffn_dim=64)
    eng = ServingEngine(ModelRunner(cfg, device="cpu", num_blocks=16), eos_id=None)
    assert len(eng.generate([1, 2, 3], 7)) == 7
    from rustral_b200.parallel.fault_tolerance import CommunicationError, StepWatchdog
    wd = StepWatchdog(0.05)
    with pytest.raises(CommunicationError):
        with wd.step():
            time.sleep(0.15)
    assert wd.overruns == 1
    with wd.step():
        pass                                                     # a step inside its limit passes


def test_tensor_alignment_of_odd_shapes():
    """Row lengths that are not multiples of any vector width give the same results as padded ones."""
    g = torch.Generator().manual_seed(1)
    for n in (1, 3, 7, 13, 31, 33, 127):
        x = torch.randn(5, n, generator=g)
        gamma, beta = torch.randn(n, generator=g), torch.randn(n, generator=g)
        ref = torch.nn.functional.layer_norm(x, (n,), gamma, beta, 1e-5)
        assert torch.allclose(ops.layer_norm(x, gamma, beta, 1e-5), ref, atol=1e-5)
        assert torch.allclose(ops.softmax(x), torch.softmax(x, -1), atol=1e-6)


# ---- edge cases -----------------------------------------------------------------------------------------------------
def test_maximum_dimensions_high_rank_and_long_rows():
    t = torch.ones(2, 1, 3, 1, 2, 1, 2, 1)
    assert T.sum_all(t) == 24.0 if hasattr(T, "sum_all") else float(t.sum()) == 24.0
    long_row = torch.zeros(1, 1 << 16)
    long_row[0, 12345] = 50.0
    p = ops.softmax(long_row)
    assert abs(float(p.sum()) - 1.0) < 1e-5 and int(p.argmax()) == 12345


def test_very_deep_networks_keep_finite_activations_and_gradients():
    layers = []
    for i in range(48):
        layers += [LinearBuilder(16, 16).with_bias().seed(i).build(BE), LayerNorm.new(BE, 16)]
    net = Sequential(*layers)
    x = torch.randn(4, 16, generator=torch.Generator().manual_seed(2), requires_grad=True)
    y = net(x, ForwardCtx.train(BE))
    y.sum().backward()
    assert torch.isfinite(y).all() and torch.isfinite(x.grad).all()
    assert all(p.tensor.grad is not None and torch.isfinite(p.tensor.grad).all() for p in net.parameters())


def test_mixed_precision_boundaries():
    """Values at the edge of bf16's range and resolution."""
    big = torch.tensor([3.0e38, -3.0e38, 1e-38, 65504.0, 65536.0])
    b = big.bfloat16()
    assert torch.isfinite(b).all() and float(b[3]) == 65536.0            # 65504 rounds up: 8 significant bits
    assert float(torch.tensor(1.0 + 2 ** -9).bfloat16()) == 1.0          # below half a unit in the last place
    assert float(torch.tensor(1.0 + 2 ** -7).bfloat16()) == 1.0 + 2 ** -7
    x = torch.full((4, 8), 300.0).bfloat16()
    s = ops.softmax(x)                                                   # exp(300) overflows unless the maximum is subtracted
    assert torch.allclose(s.float(), torch.full((4, 8), 0.125), atol=1e-3)


# ---- stress ---------------------------------------------------------------------------------------------------------
def test_rapid_allocation_and_deallocation_reuses_buffers():
    pool = TensorPool()
    seen = set()
    for i in range(500):
        t = pool.acquire((64, 64))
        seen.add(t.data_ptr())
        pool.release(t)
    assert len(seen) == 1 and pool.stats()["hits"] == 499


def test_memory_pressure_recovery():
    """After a refused oversized request the allocator serves normal requests again."""
    from rustral_b200.serve.kv_cache import PagedCache
    cache = PagedCache(8, 16, 1, 1, 8, torch.float32, "cpu")
    for round_ in range(20):
        assert not cache.allocate(100 + round_, 16 * 9)                  # more than the cache holds
        assert cache.allocate(round_, 16 * 8)
        cache.free(round_)
    assert cache.free_blocks == 8


def test_large_model_load_round_trip():
    cfg = TransformerEncoderConfig(128, 4, 4, 512, 0.0, 64)
    a = TransformerEncoder.new(BE, cfg, 2000, seed=1)
    blob = save_model(a)
    n_params = sum(p.tensor.numel() for p in a.parameters())
    assert n_params > 1_000_000 and len(blob) > 4 * n_params
    b = TransformerEncoder.new(BE, cfg, 2000, seed=2)
    load_model(b, blob)
    assert all(torch.equal(p.tensor, q.tensor) for p, q in zip(a.parameters(), b.parameters()))


def test_repeated_serialization_is_stable_and_does_not_grow():
    lin = LinearBuilder(64, 64).with_bias().seed(3).build(BE)
    first = save_model(lin)
    for _ in range(100):
        blob = save_model(lin)
        load_model(lin, blob)
    assert blob == first


def test_timeout_handling_of_a_stalled_rank():
    """A peer that stops sending heartbeats is suspected and then declared failed on the caller's clock."""
    from rustral_b200.parallel.fault_tolerance import DictStore, HealthMonitor, NodeState
    now = [0.0]
    store = DictStore()
    mons = [HealthMonitor(r, timeout_ms=1000.0, store=store, clock=lambda: now[0]) for r in range(2)]
    for m in mons:
        m.register_node(0)
        m.register_node(1)
        m.heartbeat()
    assert mons[0].check_health() == [] and mons[0].healthy_nodes() == [0, 1]
    now[0] = 1.5                                         # rank 1 is silent from here on
    mons[0].heartbeat()
    assert mons[0].check_health() == [] and mons[0].nodes[1].state is NodeState.SUSPECTED
    now[0] = 2.5
    mons[0].heartbeat()
    assert mons[0].check_health() == [1] and mons[0].nodes[1].state is NodeState.FAILED and mons[0].healthy_nodes() == [0]


# ---- performance category ---------------------------------------------------------------------------------------------
def _bench(fn, iters=5, warmup=1):
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - t0) / iters


@pytest.mark.parametrize("name,batch,i,o", [("small", 32, 64, 64), ("medium", 64, 512, 512), ("large", 64, 2048, 2048)])
def test_benchmark_linear(name, batch, i, o):
    lin = LinearBuilder(i, o).with_bias().build(BE)
    x = torch.randn(batch, i)
    t = _bench(lambda: lin(x))
    gflops = 2.0 * batch * i * o / t / 1e9
    assert lin(x).shape == (batch, o) and gflops > 0.05, f"{name}: {gflops:.2f} GFLOP/s"


def test_benchmark_conv2d_small():
    conv = Conv2d.new(BE, Conv2dConfig(8, 3, 3, in_channels=3))
    img = torch.randn(4, 3, 32, 32)
    t = _bench(lambda: conv(img))
    assert conv(img).shape == (4, 8, 32, 32) and t < 1.0


def test_benchmark_self_attention():
    q = k = v = torch.randn(2, 128, 4, 32)
    t = _bench(lambda: scaled_dot_product_attention(q, k, v, causal=True))
    assert t < 1.0


def test_benchmark_transformer_encoder_and_decoder():
    cfg = TransformerEncoderConfig(64, 4, 2, 128, 0.0, 64)
    enc = TransformerEncoder.new(BE, cfg, 500)
    dec = TransformerDecoder.new(BE, TransformerDecoderConfig(**cfg.__dict__), 500)
    ids = [[(i * 7 + j) % 500 for j in range(64)] for i in range(4)]
    ctx = ForwardCtx.inference(BE)
    te = _bench(lambda: enc.forward(ids, ctx), iters=3)
    td = _bench(lambda: dec.forward(torch.tensor(ids), ctx), iters=3)
    assert te < 2.0 and td < 2.0


def test_benchmark_embedding_lookup():
    emb = Embedding.new(BE, 10000, 128)
    ids = torch.randint(0, 10000, (64, 128))
    ctx = ForwardCtx.inference(BE)
    t = _bench(lambda: emb(ids, ctx))
    assert emb(ids, ctx).shape == (64, 128, 128) and 64 * 128 / t > 1e5          # lookups per second


def test_benchmark_end_to_end_training_pipeline():
    """Tokenise -> batch -> forward -> loss -> backward -> update, timed; the loss must fall."""
    from rustral_b200.models.config import preset
    from rustral_b200.runtime.lm_trainer import LMTrainer, TrainConfig
    cfg = preset("gpt2-test", seq_len=32)
    tr = LMTrainer(cfg, TrainConfig(global_batch=8, micro_batch=4, lr=3e-3), torch.device("cpu"))
    toks = torch.randint(0, cfg.vocab_size, (8, 33), generator=torch.Generator().manual_seed(4))
    t0 = time.perf_counter()
    losses = [tr.step(toks) for _ in range(12)]
    dt = time.perf_counter() - t0
    assert losses[-1] < losses[0] - 0.2 and dt < 60


def test_benchmark_memory_and_batch_scaling():
    """Activation memory and time grow about linearly with the batch (a quadratic blow-up would show here)."""
    lin = LinearBuilder(256, 256).with_bias().build(BE)
    prof = MemoryProfiler(capacity_bytes=1 << 40)
    sizes, times = [], []
    for b in (8, 64, 512):
        x = torch.randn(b, 256)
        with prof.track_tensor(f"b{b}", lin(x)) as tr:
            sizes.append(prof.current)
        times.append(_bench(lambda: lin(x), iters=10))
    assert sizes[1] == 8 * sizes[0] and sizes[2] == 8 * sizes[1]
    assert times[2] < 64 * times[0] * 8 + 0.05
