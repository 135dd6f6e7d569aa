"""Unit tests of public helpers by name: the flat parameter layout of the fused trainer, ZeRO-3 buckets, the dataset
cache, the operation profiler's pieces, backend capabilities, FSDP sharding helpers and activation checkpointing."""
import gzip
import hashlib
import os

import pytest
import torch

from rustral_b200.models.config import GPTConfig


def _tiny(arch="gpt2", **kw):
    base = dict(vocab_size=100, seq_len=16, n_layer=2, n_head=2, d_model=16, ffn_dim=32, arch=arch)
    base.update(kw)
    return GPTConfig(**base)


# ---------------------------------------------------------------------------------------------- flat parameter layout
def test_param_specs_put_decayed_parameters_first_on_aligned_disjoint_ranges():
    from rustral_b200.runtime.fused_gpt import ALIGN, ParamSpec, param_specs
    for arch in ("gpt2", "llama"):
        specs = param_specs(_tiny(arch))
        assert all(isinstance(s, ParamSpec) for s in specs)
        decay_flags = [s.decay for s in specs]
        assert decay_flags == sorted(decay_flags, reverse=True)          # one contiguous range per optimizer group
        end = 0
        for s in specs:
            assert s.offset % ALIGN == 0 and s.offset >= end
            end = s.offset + s.numel
        assert len({s.name for s in specs}) == len(specs)
    names = {s.name for s in param_specs(_tiny("gpt2"))}
    assert "pos_embed.embed" in names and "head.weight" not in names     # tied head, learned positions
    names = {s.name for s in param_specs(_tiny("llama"))}
    assert "head.weight" in names and "pos_embed.embed" not in names and "layers.0.ffn.gate_up.weight" in names


def test_init_flat_host_is_seeded_and_keeps_padded_vocabulary_rows_at_zero():
    from rustral_b200.runtime.fused_gpt import init_flat_host, param_specs
    cfg = _tiny()
    specs = param_specs(cfg)
    total = specs[-1].offset + specs[-1].numel
    a, b, c = (init_flat_host(cfg, specs, total, s) for s in (3, 3, 4))
    assert torch.equal(a, b) and not torch.equal(a, c)
    by = {s.name: s for s in specs}
    emb = a[by["tok_embed.embed"].offset:][:by["tok_embed.embed"].numel].view(cfg.vocab_padded, cfg.d_model)
    assert cfg.vocab_padded == 128 and float(emb[cfg.vocab_size:].abs().sum()) == 0.0 and float(emb[:cfg.vocab_size].std()) > 0.01
    ln = by["layers.1.ln2.weight"]
    assert torch.equal(a[ln.offset:ln.offset + ln.numel], torch.ones(cfg.d_model))
    wo = by["layers.0.attn.wo.weight"]
    assert float(a[wo.offset:wo.offset + wo.numel].std()) < float(emb[:cfg.vocab_size].std())    # residual projections are scaled down


def test_flat_state_round_trip_is_strict_and_leaves_the_image_alone_on_error():
    from rustral_b200.core.errors import SerializationError, ShapeMismatch
    from rustral_b200.runtime.fused_gpt import flat_to_state, init_flat_host, param_specs, state_to_flat
    cfg = _tiny("llama", n_head=4, n_kv_head=2)
    specs = param_specs(cfg)
    total = specs[-1].offset + specs[-1].numel
    host = init_flat_host(cfg, specs, total, 1)
    state = flat_to_state(cfg, specs, host)
    hd = cfg.head_dim
    assert state["layers.0.attn.wq.weight"].shape == (4 * hd, 16) and state["layers.0.attn.wk.weight"].shape == (2 * hd, 16)
    assert state["tok_embed.embed"].shape == (100, 16) and "layers.0.attn.wqkv.weight" not in state
    other = torch.zeros_like(host)
    state_to_flat(cfg, specs, state, other)
    assert flat_to_state(cfg, specs, other).keys() == state.keys()
    for k, v in flat_to_state(cfg, specs, other).items():
        assert torch.equal(v, state[k]), k
    before = other.clone()
    missing = {k: v for k, v in state.items() if k != "final_norm.weight"}
    with pytest.raises(SerializationError, match="missing"):
        state_to_flat(cfg, specs, missing, other)
    with pytest.raises(SerializationError, match="unexpected"):
        state_to_flat(cfg, specs, {**state, "extra.weight": torch.zeros(1)}, other)
    bad = {**state, "final_norm.weight": torch.zeros(17)}
    with pytest.raises((ShapeMismatch, SerializationError)):
        state_to_flat(cfg, specs, bad, other)
    assert torch.equal(other, before)


# ------------------------------------------------------------------------------------------------------ ZeRO-3 buckets
def test_zero3_buckets_place_every_parameter_once_and_shard_evenly():
    from rustral_b200.parallel.zero3 import ALIGN, Bucket, bucket_of, build_buckets
    from rustral_b200.runtime.fused_gpt import param_specs
    assert bucket_of("tok_embed.embed") == 0 and bucket_of("final_norm.weight") == 0
    assert bucket_of("layers.0.ln1.weight") == 1 and bucket_of("layers.11.ffn.fc2.bias") == 12
    cfg = _tiny()
    for world in (1, 2, 8):
        buckets, placement = build_buckets(cfg, world)
        assert len(buckets) == cfg.n_layer + 1 and all(isinstance(b, Bucket) for b in buckets)
        assert set(placement) == {s.name for s in param_specs(cfg)}
        start = 0
        for b in buckets:
            assert b.length % (world * ALIGN) == 0 and b.n_per_rank * world == b.length and b.shard_start == start
            start += b.n_per_rank
            end = 0
            for spec, off in b.specs:                                     # disjoint, aligned, decayed ones below decay_end
                assert placement[spec.name] == (b.index, off) and off % ALIGN == 0 and off >= end
                assert (off < b.decay_end) == spec.decay
                end = off + spec.numel
            assert end <= b.length
        assert buckets[1].length == buckets[2].length                    # every transformer block has the same layout


# ------------------------------------------------------------------------------------------------------ dataset cache
def test_fnv1a64_matches_the_published_test_vectors():
    from rustral_b200.data.fetch import fnv1a64
    assert fnv1a64(b"") == 0xCBF29CE484222325
    assert fnv1a64(b"a") == 0xAF63DC4C8601EC8C
    assert fnv1a64(b"foobar") == 0x85944171F73967E8


def test_fetch_url_caches_verifies_and_respects_offline_mode(tmp_path, monkeypatch):
    from rustral_b200.data.fetch import FetchError, cache_root, fetch_url, ungzip
    monkeypatch.setenv("RUSTRAL_CACHE_DIR", str(tmp_path / "cache"))
    monkeypatch.delenv("RUSTRAL_DATASET_OFFLINE", raising=False)
    monkeypatch.delenv("RUSTRAL_DATASET_SKIP_CHECKSUM", raising=False)
    assert cache_root() == str(tmp_path / "cache") and os.path.isdir(cache_root())
    src = tmp_path / "corpus.txt.gz"
    with gzip.open(src, "wb") as f:
        f.write(b"the quick brown fox\n" * 10)
    digest = hashlib.sha256(src.read_bytes()).hexdigest()
    url = "file://" + str(src)
    with pytest.raises(FetchError, match="checksum"):
        fetch_url(url, "0" * 64, "demo")
    assert not os.path.exists(os.path.join(cache_root(), "demo", "corpus.txt.gz.partial"))
    path = fetch_url(url, digest, "demo")
    assert path == os.path.join(cache_root(), "demo", "corpus.txt.gz") and open(path, "rb").read() == src.read_bytes()
    src.unlink()                                                         # served from the cache from now on
    assert fetch_url(url, digest, "demo") == path
    with pytest.raises(FetchError, match="cached file"):
        fetch_url(url, "1" * 64, "demo")
    monkeypatch.setenv("RUSTRAL_DATASET_SKIP_CHECKSUM", "1")
    assert fetch_url(url, "1" * 64, "demo") == path
    monkeypatch.setenv("RUSTRAL_DATASET_OFFLINE", "1")
    with pytest.raises(FetchError, match="OFFLINE"):
        fetch_url("file:///nonexistent/other.bin", None, "demo")
    monkeypatch.delenv("RUSTRAL_DATASET_OFFLINE")
    with pytest.raises(FetchError, match="failed"):
        fetch_url("file:///nonexistent/other.bin", None, "demo")
    out = ungzip(path, str(tmp_path / "corpus.txt"))
    assert open(out, "rb").read() == b"the quick brown fox\n" * 10 and not os.path.exists(out + ".partial")


# --------------------------------------------------------------------------------------------------- operation profiler
def test_shape_bucket_rounds_every_dimension_up_to_a_power_of_two():
    from rustral_b200.core.operation_profiler import shape_bucket
    assert shape_bucket(None) == "-" and shape_bucket(()) == "scalar"
    assert shape_bucket((1, 3, 64, 65)) == "1x4x64x128" and shape_bucket([1000]) == "1024"


def test_operation_stats_and_guard_accumulate_per_name_and_bucket():
    from rustral_b200.core.operation_profiler import DeviceType, OperationGuard, OperationProfiler, OperationStats
    st = OperationStats()
    st.record(2.0, DeviceType.CPU, "8x8")
    st.record(6.0, DeviceType.CPU, "8x8")
    st.record(1.0, DeviceType.CUDA, "16")
    assert (st.count, st.total_ms, st.min_ms, st.max_ms, st.last_ms) == (3, 9.0, 1.0, 6.0, 1.0)
    assert st.cpu_ms == 8.0 and st.gpu_ms == 1.0 and set(st.shape_buckets) == {"8x8", "16"}
    d = st.to_dict()
    assert d["count"] == 3 and abs(d["total_ms"] - 9.0) < 1e-12
    prof = OperationProfiler(use_cuda_events=False)
    with prof.guard("matmul", (5, 7)) as g:
        assert isinstance(g, OperationGuard) and g.bucket == "8x8"
        sum(range(1000))
    with prof.guard("matmul", (5, 7)):
        pass
    prof.record("softmax", 0.25)
    prof.resolve()
    top = dict((name, stats) for name, stats in prof.most_expensive_ops(5))
    assert set(top) == {"matmul", "softmax"} and top["matmul"].count == 2 and top["matmul"].shape_buckets == {"8x8": 2}
    assert prof.total_ms() >= 0.25
    prof.reset()
    assert prof.most_expensive_ops(5) == [] and prof.total_ms() == 0.0


def test_profiler_from_environment_is_off_by_default_and_reports_when_asked(monkeypatch, tmp_path, capsys):
    from rustral_b200.core.operation_profiler import OperationProfiler, finish_profile_from_env, operation_profiler_from_env
    monkeypatch.delenv("RUSTRAL_PROFILE", raising=False)
    assert operation_profiler_from_env() is None
    finish_profile_from_env(None)                                        # nothing to do, nothing printed
    assert capsys.readouterr().out == ""
    monkeypatch.setenv("RUSTRAL_PROFILE", "1")
    prof = operation_profiler_from_env()
    assert isinstance(prof, OperationProfiler)
    prof.record("add", 1.5)
    out_json = tmp_path / "profile.json"
    monkeypatch.setenv("RUSTRAL_PROFILE_EXPORT_JSON", str(out_json))
    finish_profile_from_env(prof)
    assert "add" in capsys.readouterr().out and "add" in out_json.read_text()


# ------------------------------------------------------------------------------------------------------------- backend
def test_backend_capabilities_answer_batch_precision_and_per_operation_dtype():
    from rustral_b200.core.backend import BackendCapabilities, ConvLayout, OperationType, TrainingDtype
    caps = BackendCapabilities(supports_bf16=True, supports_tensor_cores=True, max_batch_size=64,
                               recommended_training_dtype=TrainingDtype.BF16, preferred_conv_layout=ConvLayout.NHWC)
    assert caps.clamp_batch_size(1000) == 64 and caps.clamp_batch_size(0) == 1 and caps.clamp_batch_size(7) == 7
    assert caps.recommends_mixed_precision()
    assert not BackendCapabilities(supports_bf16=True).recommends_mixed_precision()          # no tensor cores
    assert caps.recommended_dtype_for_operation(OperationType.MATMUL) is TrainingDtype.BF16
    for op in (OperationType.REDUCTION, OperationType.NORMALIZATION, OperationType.SOFTMAX, OperationType.LOSS):
        assert caps.recommended_dtype_for_operation(op) is TrainingDtype.F32
    assert TrainingDtype.BF16.torch() is torch.bfloat16 and TrainingDtype.F32.torch() is torch.float32


def test_default_backend_can_be_replaced_and_initialises_parameters_from_the_seed():
    from rustral_b200.core import backend as B
    saved = B.default_backend()
    try:
        cpu = B.CpuBackend()
        B.set_default_backend(cpu)
        assert B.default_backend() is cpu and isinstance(cpu, B.Backend) and cpu.device().type == "cpu"
        a, b, c = (cpu.normal_parameter("w", (4, 5), s, 0.1) for s in (7, 7, 8))
        assert torch.equal(a.tensor, b.tensor) and not torch.equal(a.tensor, c.tensor) and a.name == "w"
        assert float(cpu.normal_parameter("z", (3,), 1, 0.0).tensor.detach().abs().sum()) == 0.0
        u = cpu.uniform_parameter("u", (1000,), 2, 0.5).tensor.detach()
        assert float(u.min()) >= -0.5 and float(u.max()) <= 0.5 and float(u.std()) > 0.2
        assert torch.equal(cpu.constant_parameter("c", (2, 2), 3.0).tensor, torch.full((2, 2), 3.0))
        assert cpu.parameter_from_vec("v", [1, 2, 3, 4, 5, 6], (2, 3)).tensor.tolist() == [[1, 2, 3], [4, 5, 6]]
        caps = cpu.capabilities()
        assert isinstance(caps, B.BackendCapabilities) and not caps.supports_tensor_cores
    finally:
        B.set_default_backend(saved)


# ---------------------------------------------------------------------------------------------------------------- FSDP
def test_shard_range_partitions_a_flat_parameter_with_sizes_that_differ_by_at_most_one():
    from rustral_b200.parallel.fsdp import shard_range
    for numel in (0, 1, 7, 64, 1001):
        for world in (1, 2, 3, 8):
            spans = [shard_range(numel, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == numel
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


def test_fsdp_config_builders_and_wrap_policy():
    from rustral_b200.nn.linear import Linear
    from rustral_b200.core.backend import CpuBackend
    from rustral_b200.parallel.fsdp import AutoWrapPolicy, FSDPCheckpoint, FSDPConfig, ShardedParameter
    cfg = FSDPConfig().with_cpu_offload().with_mixed_precision().with_bucket_size(1 << 20)
    assert cfg.cpu_offload and cfg.mixed_precision and cfg.bucket_size == 1 << 20 and cfg.shard_params and cfg.shard_grads
    lin = Linear.new(CpuBackend(), 8, 4, seed=0) if hasattr(Linear, "new") else Linear(CpuBackend(), 8, 4)
    n = sum(p.numel() for _, p in lin.named_parameters())
    assert AutoWrapPolicy(min_params=n).should_wrap(lin) and not AutoWrapPolicy(min_params=n + 1).should_wrap(lin)
    assert AutoWrapPolicy(type_names=("Linear",)).should_wrap(lin) and not AutoWrapPolicy(type_names=("Conv2d",)).should_wrap(lin)
    assert not AutoWrapPolicy().should_wrap(lin)
    assert AutoWrapPolicy(predicate=lambda m: False, type_names=("Linear",)).should_wrap(lin) is False     # the predicate decides alone
    sp = ShardedParameter("w", (4, 4), 16, 8, 16, torch.arange(8.0))
    assert sp.end - sp.start == sp.shard.numel() and sp.grad_shard is None and not sp.is_gathered
    ck = FSDPCheckpoint({"w": sp.shard}, None, rank=1, world_size=2)
    assert ck.rank == 1 and ck.world_size == 2 and ck.optimizer_state is None


# ---------------------------------------------------------------------------------------------- activation checkpointing
def test_checkpoint_config_selects_every_nth_layer():
    from rustral_b200.autograd.checkpoint import CheckpointConfig
    c = CheckpointConfig(checkpoint_every_n_layers=2)
    assert [c.should_checkpoint(i) for i in range(6)] == [False, True, False, True, False, True]
    assert not any(CheckpointConfig(enabled=False).should_checkpoint(i) for i in range(6))
    assert not any(CheckpointConfig(checkpoint_every_n_layers=0).should_checkpoint(i) for i in range(6))
    assert [CheckpointConfig(checkpoint_every_n_layers=3).should_checkpoint(i) for i in range(5)] == [False, True, False, False, True]


def test_checkpoint_segment_recomputes_in_backward_and_gives_the_same_gradients():
    from rustral_b200.autograd.checkpoint import CheckpointedSegment, checkpoint_segment
    torch.manual_seed(0)
    w = torch.randn(6, 6, requires_grad=True)
    x = torch.randn(4, 6, requires_grad=True)
    calls = []

    def block(t):
        calls.append(1)
        return torch.tanh(t @ w).pow(2)

    y_plain = block(x)
    gx, gw = torch.autograd.grad(y_plain.sum(), (x, w))
    calls.clear()
    y = checkpoint_segment(block, x, parameters=(w,))
    assert len(calls) == 1 and torch.equal(y, y_plain) and y.grad_fn is not None
    cx, cw = torch.autograd.grad(y.sum(), (x, w))
    assert len(calls) == 2                                              # the forward ran again inside the backward pass
    assert torch.allclose(cx, gx, atol=1e-6) and torch.allclose(cw, gw, atol=1e-6)
    seg = CheckpointedSegment(x, lambda t: t * 2, input_id=3, output_id=4)
    assert torch.equal(seg.recompute(), x.detach() * 2) and seg.saved_bytes() == 4 * 6 * 4 and not seg.input_value.requires_grad


def test_checkpoint_manager_wraps_layers_and_memory_stats_show_the_saving():
    from rustral_b200.autograd.checkpoint import (CheckpointConfig, CheckpointedTransformerLayer, CheckpointManager, MemoryStats,
                                                  checkpoint_model)

    class Scale:
        def __init__(self, k):
            self.k = k

        def __call__(self, x, ctx):
            return x * self.k

        def parameters(self):
            return []

        def named_parameters(self):
            return []

    layers = [Scale(2.0), Scale(3.0), Scale(5.0)]
    wrapped = CheckpointManager(CheckpointConfig(checkpoint_every_n_layers=2)).wrap(layers)
    assert [type(l) for l in wrapped] == [CheckpointedTransformerLayer] * 3 and [l.layer_idx for l in wrapped] == [0, 1, 2]
    x = torch.ones(2, 2, requires_grad=True)
    h = x
    for l in wrapped:
        h = l(h, None)
    h.sum().backward()
    assert torch.equal(h.detach(), torch.full((2, 2), 30.0)) and torch.equal(x.grad, torch.full((2, 2), 30.0))
    assert len(checkpoint_model(layers)) == 3 and checkpoint_model(layers)[1].config.checkpoint_every_n_layers == 2
    m = MemoryStats.calculate(num_layers=12, batch=8, seq=1024, d_model=768, ffn_dim=3072, every_n=2)
    per_layer = 8 * 1024 * (8 * 768 + 2 * 3072) * 2
    assert m.without_bytes == 12 * per_layer and m.with_bytes < m.without_bytes and 0.3 < m.savings < 0.5
    assert MemoryStats.calculate(12, 8, 1024, 768, 3072, every_n=100).with_bytes > m.with_bytes   # fewer checkpoints keep more


# ------------------------------------------------------------------------------------------------------ memory profiler
def test_memory_profiler_tracks_allocations_by_tag_and_grades_the_oom_risk():
    from rustral_b200.core.memory_profiler import AllocationEvent, AllocationTracker, MemoryProfiler, OOMRisk, OomRisk, global_profiler
    p = MemoryProfiler(capacity_bytes=1000)
    h1 = p.alloc("weights", 300)
    h2 = p.alloc("activations", 300)
    assert (p.current, p.peak, p.by_tag["weights"]) == (600, 600, 300)
    assert p.predict_oom_risk() == OOMRisk.MEDIUM and p.predict_oom_risk(200) == OOMRisk.HIGH and p.predict_oom_risk(400) == OOMRisk.CRITICAL
    assert OomRisk(p.predict_oom_risk()) is OomRisk.MEDIUM
    p.free(h2)
    p.free(h2)                                                            # a second free of the same handle changes nothing
    assert (p.current, p.peak) == (300, 600) and p.predict_oom_risk() == OOMRisk.LOW
    assert [(e.kind, e.tag, e.nbytes) for e in p.events] == [("alloc", "weights", 300), ("alloc", "activations", 300), ("free", "activations", 300)]
    assert all(isinstance(e, AllocationEvent) for e in p.events)
    assert [(h, tag, n) for h, tag, n in p.find_leaks()] == [(h1, "weights", 300)] and p.find_leaks(older_than_s=3600) == []
    with AllocationTracker(p, "scratch", 50) as t:
        assert p.current == 350 and t.h
    assert p.current == 300 and t.h == 0
    t.release()                                                           # idempotent
    assert p.current == 300
    tr = p.track_tensor("batch", torch.zeros(4, 4))
    assert p.by_tag["batch"] == 64
    tr.release()
    assert p.by_tag["batch"] == 0
    assert '"tag": "scratch"' in p.export_timeline()
    assert global_profiler() is global_profiler()


# ------------------------------------------------------------------------------------------------------------ dashboard
def test_sparkline_and_progress_bar_render_fixed_width_text():
    from rustral_b200.utils.tui import progress_bar, sparkline
    assert sparkline([]) == "" and sparkline([float("nan"), None]) == ""
    s = sparkline([0, 1, 2, 3], width=40)
    assert len(s) == 4 and s[0] == "▁" and s[-1] == "█" and list(s) == sorted(s)
    assert len(sparkline(range(100), width=10)) == 10 and set(sparkline([5, 5, 5])) == {"▁"}
    assert progress_bar(0, 10, width=10) == "░" * 10 + "   0.0%"
    assert progress_bar(5, 10, width=10) == "█" * 5 + "░" * 5 + "  50.0%"
    assert progress_bar(20, 10, width=4) == "████ 100.0%" and progress_bar(1, 0, width=4).endswith("  0.0%")


def test_tui_metrics_backend_routes_scalars_into_the_dashboard_by_name():
    from rustral_b200.metrics import ScalarMetric
    from rustral_b200.utils.tui import LeakWarning, TrainingDashboard, TuiMetricsBackend
    be = TuiMetricsBackend()
    dash = be.dashboard()
    assert isinstance(dash, TrainingDashboard)
    be.log_scalar(ScalarMetric("train/loss", 2.5, 7, 0.0))
    be.log_scalar(ScalarMetric("val_accuracy", 0.75, 8, 0.0))
    be.log_scalar(ScalarMetric("lr", 3e-4, 9, 0.0))
    be.log_scalar(ScalarMetric("grad_norm", 1.0, 10, 0.0))               # not a dashboard series: only the step moves
    assert dash.losses == [2.5] and dash.accuracies == [0.75] and dash.step == 10
    be.log_scalar(ScalarMetric("loss", float("inf"), 11, 0.0))
    assert len(dash.losses) == 2
    shared = TrainingDashboard("shared")
    assert TuiMetricsBackend(shared).dashboard() is shared
    w = LeakWarning("kv", 1 << 20, 12.0)
    assert (w.tag, w.nbytes, w.allocation_count) == ("kv", 1 << 20, 1)


# ---------------------------------------------------------------------------------------------------- context parallel
def test_sequence_sharding_and_context_parallel_bookkeeping():
    from rustral_b200.parallel.process_group import DistributedError, ProcessGroup
    from rustral_b200.parallel.sequence_parallel import (CommunicationStats, ContextParallel, ContextParallelConfig, DynamicLoadBalancer,
                                                         compute_sequence_sharding)
    assert compute_sequence_sharding(16, 4) == [(0, 4), (4, 8), (8, 12), (12, 16)]
    cfg = ContextParallelConfig(num_devices=4, sequence_length=32768, block_size=4096)
    cfg.validate()
    assert cfg.tokens_per_device() == 8192 and cfg.striped and cfg.causal
    with pytest.raises(DistributedError, match="divisible"):
        ContextParallelConfig(num_devices=3, sequence_length=32768).validate()
    with pytest.raises(DistributedError, match="block_size"):
        ContextParallelConfig(num_devices=4, sequence_length=4 * 6000, block_size=4096).validate()
    ContextParallelConfig(num_devices=4, sequence_length=4 * 1000, block_size=4096).validate()     # shorter than one block is fine
    cp = ContextParallel(ProcessGroup.new_single_process(), ContextParallelConfig(num_devices=1, sequence_length=8, block_size=8))
    x = torch.arange(16.0).view(1, 8, 2)
    assert torch.equal(cp.shard_input(x), x)
    st = cp.communication_stats(kv_heads=8, head_dim=128, batch=2)
    assert isinstance(st, CommunicationStats) and st.steps == 0 and st.total_bytes == 0 and st.kv_bytes_per_step == 8 * 2 * 8 * 128 * 2 * 2
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 8, 2, 4) for _ in range(3))
    out = cp.forward(q, k, v)
    ref = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True).transpose(1, 2)
    assert torch.allclose(out.float(), ref, atol=1e-5)
    lb = DynamicLoadBalancer(4, threshold=1.2)
    assert lb.overloaded() == []
    for r, t in enumerate((1.0, 1.0, 1.0, 2.0)):
        lb.report(r, t)
    assert lb.overloaded() == [3]
    lb.report(3, 1.1)
    assert lb.overloaded() == []


# ------------------------------------------------------------------------------------------------------ fault tolerance
def test_fault_records_and_the_in_memory_checkpoint_store():
    from rustral_b200.parallel.fault_tolerance import (CheckpointStore, FaultStats, MembershipChange, MemoryCheckpointStore, NodeInfo,
                                                       NodeState)
    n = NodeInfo(3)
    assert n.state is NodeState.HEALTHY and n.last_checkpoint == -1 and n.last_heartbeat == 0.0
    ch = MembershipChange("shrink", [2], new_world_size=3, new_rank=2)
    assert ch.kind == "shrink" and ch.ranks == [2] and MembershipChange("none").ranks == []
    assert FaultStats() == FaultStats(0, 0, 0, 0)
    for m in ("save", "load", "latest"):
        with pytest.raises(NotImplementedError):
            getattr(CheckpointStore(), m)(*([0, {}] if m == "save" else [0] if m == "load" else []))
    store = MemoryCheckpointStore()
    assert isinstance(store, CheckpointStore) and store.latest() is None
    state = {"w": torch.ones(2)}
    store.save(10, state)
    state["w"].zero_()                                                    # the store keeps its own copy
    store.save(20, state)
    assert store.latest() == 20 and torch.equal(store.load(10)["w"], torch.ones(2)) and torch.equal(store.load(20)["w"], torch.zeros(2))


# ------------------------------------------------------------------------------------------------------------------ MoE
def test_top_k_gating_returns_normalised_weights_and_the_load_balance_loss():
    from rustral_b200.core import CpuBackend, ForwardCtx
    from rustral_b200.nn.moe import GatingOutput, MoEConfig, MoEOutput, MoEStats, TopKGating
    cfg = MoEConfig(d_model=8, num_experts=4, expert_dim=16, top_k=2)
    gate = TopKGating.new(CpuBackend(), cfg, seed=1)
    torch.manual_seed(0)
    x = torch.randn(32, 8)
    g = gate.forward(x, ForwardCtx(CpuBackend()))
    assert isinstance(g, GatingOutput) and g.indices.shape == (32, 2) and g.weights.shape == (32, 2) and g.probs.shape == (32, 4)
    logits = x @ gate.gate_proj.tensor.detach().t()
    probs = torch.softmax(logits, -1)
    top_p, top_i = probs.topk(2, -1)
    assert torch.equal(g.indices.long().sort(-1).values, top_i.sort(-1).values)
    assert torch.allclose(g.probs, probs, atol=1e-6) and torch.allclose(g.weights.sum(-1), torch.ones(32), atol=1e-5)
    f = torch.bincount(top_i.reshape(-1), minlength=4).float() / 64
    assert abs(float(g.aux_loss) - float((f * probs.mean(0)).sum() * 4)) < 1e-6
    assert [n for n, _ in gate.named_parameters()] == ["gate_proj"]
    out = MoEOutput(torch.zeros(2, 8), torch.tensor(0.5))
    stats = MoEStats([16, 16, 16, 16], 1.0, 0)
    assert out.output.shape == (2, 8) and float(out.aux_loss) == 0.5 and sum(stats.tokens_per_expert) == 64 and stats.dropped_tokens == 0


# ------------------------------------------------------------------------------------------------------ hub and layers
def test_hub_url_and_loading_hub_weights_from_the_cache(tmp_path, monkeypatch):
    from rustral_b200.core import CpuBackend
    from rustral_b200.nn import Linear
    from rustral_b200.utils.hf import HfError, download_state_dict, hub_url, load_from_hub, save_state_dict_to_file
    assert hub_url("org/model") == "https://huggingface.co/org/model/resolve/main/model.safetensors"
    assert hub_url("org/model", "v2", "config.json") == "https://huggingface.co/org/model/resolve/v2/config.json"
    monkeypatch.setenv("RUSTRAL_CACHE_DIR", str(tmp_path))
    monkeypatch.setenv("RUSTRAL_DATASET_OFFLINE", "1")
    with pytest.raises(HfError) as e:
        download_state_dict("org/absent")
    assert e.value.kind == "hub"
    d = tmp_path / "hf" / "org--model" / "main"
    d.mkdir(parents=True)
    lin = Linear.new(CpuBackend(), 4, 3, seed=5) if hasattr(Linear, "new") else Linear(CpuBackend(), 4, 3)
    names = [n for n, _ in lin.named_parameters()]
    want = {n: torch.full(tuple(p.tensor.shape), float(i + 1)) for i, (n, p) in enumerate(lin.named_parameters())}
    save_state_dict_to_file({("model." + k): v for k, v in want.items()} | {"model.unused": torch.zeros(1)}, str(d / "model.safetensors"))
    assert set(download_state_dict("org/model")) == {"model." + n for n in names} | {"model.unused"}
    load_from_hub(lin, "org/model", key_map=lambda k: None if k.endswith("unused") else k[len("model."):])
    for n, p in lin.named_parameters():
        assert torch.equal(p.tensor.detach(), want[n]), n
    (d / "model.safetensors").write_bytes(b"not a safetensors file")
    with pytest.raises(HfError) as e:
        download_state_dict("org/model")
    assert e.value.kind == "tensor"


def test_positional_encoding_adds_the_sinusoid_table_and_checks_the_length():
    import math
    from rustral_b200.core import CpuBackend, ForwardCtx, InvalidArgument
    from rustral_b200.nn.transformer import PositionalEncoding
    pe = PositionalEncoding(8, max_len=16)
    ctx = ForwardCtx(CpuBackend())
    y = pe.forward(torch.zeros(2, 5, 8), ctx)
    assert y.shape == (2, 5, 8) and torch.equal(y[0], y[1])
    for pos in (0, 3):
        for i in (0, 2):
            angle = pos / (10000.0 ** (2 * i / 8))
            assert abs(float(y[0, pos, 2 * i]) - math.sin(angle)) < 1e-6 and abs(float(y[0, pos, 2 * i + 1]) - math.cos(angle)) < 1e-6
    x = torch.randn(1, 4, 8, requires_grad=True)
    pe.forward(x, ctx).sum().backward()
    assert torch.equal(x.grad, torch.ones_like(x))                        # the table is a constant
    with pytest.raises(InvalidArgument, match="max_len"):
        pe.forward(torch.zeros(1, 17, 8), ctx)


def test_scheduler_records_have_the_documented_fields():
    from rustral_b200.serve.scheduler import Batch, RequestState, SchedulerStats
    assert [s.name for s in RequestState] == ["WAITING", "PREFILL", "GENERATING", "PAUSED", "COMPLETED"]
    b = Batch([1, 2], [[5, 6, 7], [9]], [3, 8], [[0], [1]], [True, False])
    assert len(b.request_ids) == len(b.input_ids) == len(b.seq_lens) == len(b.block_tables) == len(b.is_prefill) == 2
    s = SchedulerStats()
    assert (s.completed, s.preempted, s.admitted, s.total_generated, s.total_latency) == (0, 0, 0, 0, 0.0)


# ------------------------------------------------------------------------------------------------------ MoE primitives
def _routing_case(T=24, E=4, k=2, seed=0):
    from rustral_b200.ops import moe as M
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    idx, w, probs = M.route(logits, k, True)
    return M, logits, idx, w, probs


def test_moe_plan_groups_slots_by_expert_on_128_row_segments():
    M, _, idx, _, _ = _routing_case()
    pl = M.plan(idx, 4)
    assert isinstance(pl, M.MoEPlan) and pl.k == 2 and pl.num_experts == 4 and pl.max_rows % 128 == 0
    assert pl.counts.tolist() == torch.bincount(idx.reshape(-1).long(), minlength=4).tolist() and int(pl.counts.sum()) == 48
    assert all(int(o) % 128 == 0 for o in pl.offsets) and int(pl.offsets[0]) == 0
    flat = idx.reshape(-1).long()
    for s in range(48):                                                   # every slot lands inside its expert's segment
        e, pos = int(flat[s]), int(pl.slot_pos[s])
        assert int(pl.offsets[e]) <= pos < int(pl.offsets[e]) + int(pl.counts[e]) and int(pl.row_slot[pos]) == s
    assert int((pl.row_slot >= 0).sum()) == 48 and len(set(pl.slot_pos.tolist())) == 48
    ntiles = int(pl.num_tiles)
    assert ntiles == int(pl.offsets[-1]) // 128 and pl.tile_expert[:ntiles].tolist() == sorted(pl.tile_expert[:ntiles].tolist())


def test_grouped_gemm_and_its_gradients_follow_the_per_slot_definition():
    M, _, idx, _, _ = _routing_case()
    pl = M.plan(idx, 4)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(24, 8, generator=g)
    W = torch.randn(4, 6, 8, generator=g)
    xp = M.gather(x, pl)
    y = M.grouped_gemm(xp, W, pl)
    assert y.shape == (pl.max_rows, 6)
    flat = idx.reshape(-1).long()
    for s in (0, 7, 23, 47):
        assert torch.allclose(y[int(pl.slot_pos[s])], x[s // 2] @ W[int(flat[s])].t(), atol=1e-5)
    back = M.grouped_gemm(y, W, pl, b_mn=True)                           # dgrad form: rows times W[e] itself
    s = 5
    assert torch.allclose(back[int(pl.slot_pos[s])], (x[s // 2] @ W[int(flat[s])].t()) @ W[int(flat[s])], atol=1e-4)
    dyp = torch.zeros(pl.max_rows, 6)
    dyp[pl.slot_pos.long()] = torch.randn(48, 6, generator=g)
    dW = M.grouped_wgrad(dyp, xp, pl)
    ref = torch.zeros(4, 6, 8)
    for s in range(48):
        ref[int(flat[s])] += torch.outer(dyp[int(pl.slot_pos[s])], x[s // 2])
    assert torch.allclose(dW, ref, atol=1e-4)
    twice = M.grouped_wgrad(dyp, xp, pl, out=dW.clone(), accumulate=True)
    assert torch.allclose(twice, 2 * ref, atol=1e-4)
    dy = torch.randn(24, 6, generator=g)
    dw = M.weight_grad(dy, y, pl)
    assert dw.shape == (24, 2) and abs(float(dw[3, 1]) - float(dy[3] @ y[int(pl.slot_pos[7])])) < 1e-4


@pytest.mark.parametrize("renorm", [True, False])
def test_route_backward_equals_autograd_through_softmax_top_k_and_the_balance_loss(renorm):
    from rustral_b200.ops import moe as M
    T, E, k, scale = 16, 4, 2, 0.3
    g = torch.Generator().manual_seed(2)
    logits = torch.randn(T, E, generator=g, requires_grad=True)
    idx, w, probs = M.route(logits.detach(), k, renorm)
    dw = torch.randn(T, k, generator=g)
    counts = torch.bincount(idx.reshape(-1).long(), minlength=E)
    p = torch.softmax(logits, -1)
    top = p.gather(1, idx.long())
    wt = top / top.sum(-1, keepdim=True) if renorm else top
    assert torch.allclose(wt.detach(), w, atol=1e-6)
    loss = (wt * dw).sum() + scale * E * ((counts.float() / (T * k)) * p.mean(0)).sum()
    ref, = torch.autograd.grad(loss, logits)
    got = M.route_backward(probs, idx, w, dw, counts.to(torch.int32), renorm, scale)
    assert torch.allclose(got, ref, atol=1e-5)


# -------------------------------------------------------------------------------------------------------- data parallel
def test_bucketize_keeps_order_and_never_splits_a_tensor():
    from rustral_b200.parallel.data_parallel import bucketize
    ts = [torch.zeros(n) for n in (10, 10, 30, 5, 100, 1)]
    b = bucketize(ts, bucket_bytes=100)                                   # 25 floats per bucket
    assert [[t.numel() for t in bk] for bk in b] == [[10, 10], [30], [5], [100], [1]]
    assert [t for bk in b for t in bk] == ts or all(x is y for x, y in zip([t for bk in b for t in bk], ts))
    assert bucketize([]) == [] and len(bucketize(ts)) == 1


def test_gradient_accumulator_averages_over_micro_steps_and_ranks():
    from rustral_b200.parallel.data_parallel import GradientAccumulator, all_reduce_gradients
    from rustral_b200.parallel.process_group import ProcessGroup
    acc = GradientAccumulator(ProcessGroup.new_single_process())
    acc.accumulate({"w": torch.tensor([2.0, 4.0]), "b": torch.tensor([1.0])})
    acc.accumulate({"w": torch.tensor([4.0, 0.0]), "b": torch.tensor([3.0])})
    out = acc.all_reduce()
    assert acc.steps == 2 and out["w"].tolist() == [3.0, 2.0] and out["b"].tolist() == [2.0]
    acc.reset()
    assert acc.steps == 0 and acc.acc == {}
    g = [torch.tensor([1.0, 2.0])]
    all_reduce_gradients(ProcessGroup.new_single_process(), g)
    assert g[0].tolist() == [1.0, 2.0]                                    # one rank: the average is the value itself
    import threading
    res = [None, None]

    def body(pg):
        grads = [torch.full((3,), float(pg.rank + 1)), torch.full((2,), 10.0 * (pg.rank + 1))]
        all_reduce_gradients(pg, grads, average=True, bucket_bytes=8)
        res[pg.rank] = [t.tolist() for t in grads]

    threads = [threading.Thread(target=body, args=(pg,)) for pg in ProcessGroup.new_threaded(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=30)
    assert res[0] == res[1] == [[1.5] * 3, [15.0] * 2]


# ------------------------------------------------------------------------------------------------------------ 3-D mesh
def test_3d_config_validates_the_world_size_and_layers_follow_the_pipeline_coordinate():
    from rustral_b200.parallel.parallelism_3d import Parallel3DConfig
    from rustral_b200.parallel.process_group import DistributedError
    c = Parallel3DConfig(dp=2, tp=2, pp=2)
    assert c.total_gpus() == 8
    c.validate(8)
    with pytest.raises(DistributedError):
        c.validate(4)
    assert Parallel3DConfig().total_gpus() == 1


# -------------------------------------------------------------------------------------------------------- small pieces
def test_wants_grad_follows_autograd_state():
    from rustral_b200 import _native as N
    a, b = torch.zeros(2), torch.zeros(2, requires_grad=True)
    assert not N.wants_grad(a, None) and N.wants_grad(a, b, None)
    with torch.no_grad():
        assert not N.wants_grad(a, b)
    assert isinstance(N.have_kernels(), bool)


def test_safetensors_error_types_and_state_tensor_record():
    from rustral_b200.io import safetensors_io as st
    for cls in (st.SafeTensorError, st.ShapeMismatchError, st.MissingTensor):
        assert issubclass(cls, st.IoError)
    t = st.StateTensor((2, 2), "F32", torch.zeros(2, 2))
    assert t.shape == (2, 2) and t.dtype == "F32" and t.data.numel() == 4


def test_registry_lookup_and_sst2_record():
    from rustral_b200.data.corpora import Sst2Example
    from rustral_b200.utils.model_zoo import Registry, RegistryEntry
    e = RegistryEntry("gpt2-small", "openai-community/gpt2", "main", "supported", "", "examples/load_gpt2.py")
    r = Registry("1", [e])
    assert r.get("gpt2-small") is e and r.get("absent") is None
    ex = Sst2Example("a fine film", 1)
    assert (ex.text, ex.label) == ("a fine film", 1)


def test_lr_scheduler_base_counts_steps_and_drives_an_attached_optimizer():
    from rustral_b200.optim.lr_scheduler import LRScheduler

    class Halving(LRScheduler):
        def get_lr(self, step):
            return 1.0 / (2 ** step)

    class Opt:
        lr = 0.0

        def set_lr(self, v):
            self.lr = v

    s = Halving()
    assert s.current_lr() == 1.0
    assert s.step() == 0.5 and s.step() == 0.25 and s.current_lr() == 0.25
    s.reset()
    assert s.current_lr() == 1.0 and isinstance(s.name(), str)
    with pytest.raises(NotImplementedError):
        LRScheduler().get_lr(0)


def test_cpu_forms_of_the_copy_and_cast_helpers():
    from rustral_b200.ops.elementwise import strided_copy
    from rustral_b200.ops.optim import cast_f32_to_bf16
    src = torch.arange(24.0).view(4, 6)[:, 1:4]                           # row pitch 6, width 3
    dst = torch.zeros(4, 8)[:, 2:5]
    out = strided_copy(src, dst)
    assert torch.equal(dst, src) and (out is dst or out is None or torch.equal(out, src))
    x = torch.tensor([1.0, 1.0 + 2 ** -9, 3.14159, -2.5e-3])
    y = cast_f32_to_bf16(x)
    assert y.dtype == torch.bfloat16 and torch.equal(y, x.to(torch.bfloat16))
    z = torch.empty(4, dtype=torch.bfloat16)
    assert cast_f32_to_bf16(x, z) is z and torch.equal(z, y)
