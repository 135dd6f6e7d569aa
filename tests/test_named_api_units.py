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
        u = cpu.uniform_parameter("u", (1000,), 2, 0.5).tensor
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
