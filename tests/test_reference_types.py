"""The typed results, configurations and errors that carry the reference's names: each does the job its counterpart does
there (field names as in the reference; the file / line of each is in the class's docstring)."""
import io
import json

import pytest
import torch

from rustral_b200.core import (CpuBackend, DType, ForwardCtx, FusionTestConfig, FusionTestHarness, MatmulDim, MemoryProfiler,
                               NumericsError, NumericsValidator, Op, OperationProfiler, OomRisk, OpType, PatternMatcher, PoolStats,
                               ProfilingHooks, ShapeBucket, ShapeExt, TensorPool, TensorShape)

BE = CpuBackend()


def test_memory_snapshot_summary_and_risk_enum():
    mem = MemoryProfiler(capacity_bytes=1000)
    a = mem.alloc("w", 300)
    b = mem.alloc("act", 200)
    snap = mem.snapshot("peak")
    assert (snap.total_allocated, snap.peak_allocated, snap.num_allocations, snap.by_tag) == (500, 500, 2, {"w": 300, "act": 200})
    assert snap["current"] == 500 and snap["label"] == "peak"
    mem.free(b)
    s = mem.summary()
    assert (s.current_bytes, s.peak_bytes, s.total_allocations, s.total_deallocations, s.active_count) == (300, 500, 2, 1, 1) and s.duration >= 0
    assert OomRisk(mem.predict_oom_risk(500)) is OomRisk.HIGH and OomRisk.CRITICAL.as_str() == "critical"
    mem.reset()
    assert mem.summary().total_allocations == 0 and mem.find_leaks() == [] and a


def test_shape_buckets_hooks_and_snapshot_rows():
    assert [MatmulDim.from_size(n) for n in (255, 256, 512, 513, 2047, 2048, 8191, 8192)] == [
        MatmulDim.TINY, MatmulDim.SMALL, MatmulDim.SMALL, MatmulDim.MEDIUM, MatmulDim.MEDIUM, MatmulDim.LARGE, MatmulDim.LARGE, MatmulDim.XLARGE]
    assert ShapeBucket.from_dims([32, 768]).kind == "medium" and ShapeBucket.from_dims([4, 9000, 2]).kind == "xlarge"
    mm = ShapeBucket.from_matmul_dims(128, 3072, 768)
    assert (mm.m, mm.n, mm.k) == (MatmulDim.TINY, MatmulDim.LARGE, MatmulDim.MEDIUM) and str(mm) == "matmul[tiny,large,medium]"
    assert mm == ShapeBucket.from_matmul_dims(200, 4000, 1000) and hash(mm) == hash(ShapeBucket.from_matmul_dims(200, 4000, 1000))
    prof = OperationProfiler(use_cuda_events=False).with_hooks(ProfilingHooks(shape_bucket_recording=False))
    with prof.guard("op", (3, 5)):
        pass
    with prof.guard("op", (300, 500)):
        pass
    assert prof.stats["op"].shape_buckets == {"-": 2}                      # all calls share one bucket
    rows = prof.snapshot().rows()
    assert rows[0].name == "op" and rows[0].count == 2 and rows[0].device_type == "cpu" and rows[0].max_ms >= rows[0].avg_ms
    off = OperationProfiler(use_cuda_events=False).with_hooks(ProfilingHooks.none())
    with off.guard("op", (1,)):
        pass
    assert off.stats == {} and ProfilingHooks.all().memory_tracking


def test_pool_stats_and_validation_result_and_numerics_error():
    pool = TensorPool()
    for shape in ((16, 16), (16, 16), (20, 20)):
        pool.release(torch.zeros(shape))
    st = pool.pool_stats()
    assert isinstance(st, PoolStats) and (st.total_tensors, st.unique_shapes, st.total_memory_bytes) == (3, 2, (256 + 256 + 400) * 4)
    out = io.StringIO()
    pool.print_stats(out)
    assert "total tensors: 3" in out.getvalue()
    v = NumericsValidator()
    ref = torch.linspace(1, 2, 100)
    r = v.validate(ref + 1e-7, ref)
    assert r.passed and r.num_violations == 0 and r.total_elements == 100 and r.violation_rate() == 0.0
    bad = ref.clone(); bad[:10] += 0.1
    r = v.validate(bad, ref)
    assert not r.passed and r.violation_rate() == pytest.approx(10.0) and r.max_abs_diff == pytest.approx(0.1, rel=1e-3)
    with pytest.raises(NumericsError) as e:
        v.check(bad, ref, what="probe")
    assert e.value.kind == "tolerance_exceeded" and e.value.result.num_violations == 10 and "10 of 100" in str(e.value)
    with pytest.raises(NumericsError) as e:
        v.check(ref[:5], ref)
    assert e.value.kind == "length_mismatch"
    nan = ref.clone(); nan[0] = float("nan")
    with pytest.raises(NumericsError) as e:
        v.check(nan, ref)
    assert e.value.kind == "nan"
    assert v.check(ref, ref, DType.F32).passed


def test_op_records_chain_only_when_shapes_agree_and_fusion_suite_aggregates():
    ops = [Op(OpType.MATMUL, [[4, 8], [8, 16]], [4, 16]), Op(OpType.ADD_BIAS, [[4, 16], [16]], [4, 16]), Op(OpType.GELU, [[4, 16]], [4, 16]),
           Op(OpType.MATMUL, [[4, 16], [16, 2]], [4, 2]), Op(OpType.ADD_BIAS, [[9, 9], [9]], [9, 9])]      # the last bias add reads something else
    hits = PatternMatcher().find_in_ops(ops)
    assert [(i, n, p.value) for i, n, p in hits] == [(0, 3, "matmul_bias_gelu")]
    assert OpType.of("gelu") is OpType.GELU and OpType.of("bias_add") is OpType.ADD_BIAS and OpType.of("conv") is OpType.UNKNOWN
    h = FusionTestHarness(repeats=2, config=FusionTestConfig(strict_numerics=True, num_random_cases=3))
    x = torch.randn(8, 8, generator=torch.Generator().manual_seed(0))
    suite = h.run_suite("demo", [("same", lambda: x + 1, lambda: 1 + x), ("wrong", lambda: x, lambda: x * 1.5)])
    assert (suite.total_tests, suite.passed_tests, suite.all_passed()) == (2, 1, False) and suite.avg_speedup > 0
    assert "demo: 1/2 passed" in str(suite)
    buf = io.StringIO(); suite.print_summary(buf)
    assert "wrong: FAILED" in buf.getvalue()
    rnd = h.run_random_cases("rand", lambda s: ((lambda: torch.full((4,), float(s))), (lambda: torch.full((4,), float(s)))))
    assert rnd.total_tests == 3 and rnd.all_passed()
    assert ShapeExt.elem_count((2, 3, 4)) == 24 and ShapeExt.elem_count(()) == 1
    assert TensorShape.shape_of(torch.zeros(2, 5)) == (2, 5) and TensorShape.shape_of(BE.constant_parameter("p", (3,), 0.0)) == (3,)
    with pytest.raises(TypeError):
        TensorShape.shape_of(3.0)


def test_tuner_types_and_kernel_config():
    from rustral_b200 import tune
    from rustral_b200.tune import (AlgorithmConfig, AutoTuner, BlockSize, CacheStats, ConfigCache, KernelConfig, MatmulAlgorithm,
                                   MatmulDimBucket, MemoryConfig, TunerConfig, TunerStats, TunerStrategy, WorkgroupConfig)
    assert MatmulDimBucket.from_size(512) is MatmulDimBucket.SMALL and str(MatmulDimBucket.from_size(9000)) == "XLarge"
    assert WorkgroupConfig(32, 32, 1).is_valid() and not WorkgroupConfig(64, 32, 1).is_valid() and WorkgroupConfig().total_threads() == 256
    assert BlockSize.square(64).is_valid() and not BlockSize(512, 64, 64).is_valid() and BlockSize(128, 192, 64).is_tcgen05_tile()
    assert not BlockSize(128, 100, 64).is_tcgen05_tile() and MemoryConfig(True, 300 * 1024).fits_sm100() is False
    k = KernelConfig.default_for("matmul")
    assert k.is_valid() and k.algorithm == AlgorithmConfig.matmul(MatmulAlgorithm.TCGEN05_ONE_CTA) and k.block_size() == BlockSize(128, 256, 64)
    assert k.to_gemm_plan() == {"block_n": 256, "splits": 0, "group_m": 8}
    k.params.update(tile_n=100, splits=4)
    assert k.to_gemm_plan()["block_n"] == 128 and k.to_gemm_plan()["splits"] == 4        # 100 is rounded to a width the kernel has
    assert KernelConfig.default_for("attention").algorithm.value == (True, 128, 128) and KernelConfig.default_for("nope") == KernelConfig()
    with pytest.raises(ValueError):
        KernelConfig.default_for("reduce").to_gemm_plan()
    assert k.cache_key() != KernelConfig.default_matmul().cache_key() and "wg=320x1x1" in k.cache_key()
    assert TunerStrategy is tune.Strategy and issubclass(tune.GridSearch, tune.SearchStrategy)

    class K(tune.TunableKernel):
        kernel_id, host_timed = "toy", True

        def config_space(self):
            return tune.ConfigSpace({"a": [1, 2, 3]})

        def with_config(self, c):
            return lambda: sum(range(200 * c["a"]))
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        t = AutoTuner(TunerConfig.ci_safe(), ConfigCache(d + "/c.json", "cpu"))
        t.config.device_id = "cpu"
        t.tune(K()); t.tune(K())
        st = t.stats
        assert isinstance(st, TunerStats) and st.total_tunings == 1 and st.cache_hits == 1 and st.cache_misses == 1 and st.hit_rate() == 0.5
        assert st["tuned"] == 1 and st.total_configs_tried >= 2 and st.total_tuning_time > 0
        cs = t.cache.stats()
        assert isinstance(cs, CacheStats) and cs.total_entries == 1 and cs.by_device == {"cpu": 1} and cs.cache_path.endswith("c.json")
        buf = io.StringIO(); st.print(buf); cs.print(buf)
        assert "cache hit rate: 50.0 %" in buf.getvalue() and "total entries: 1" in buf.getvalue()


def test_nn_records_states_predictions_assignments_and_routing():
    from rustral_b200.nn import (BidirectionalOutput, BidirectionalRnn, BinaryReadout, EncoderDecoderConfig, ExpertChoiceConfig,
                                 ExpertChoiceRouter, GruCell, GruConfig, GruState, LstmCell, LstmConfig, LstmState, MultiReadout,
                                 ReadoutConfig, SharedExpertConfig, SharedExpertLayer, TransformerEncoderDecoder)
    ctx = ForwardCtx.inference(BE)
    cell = LstmCell.new(BE, 4, 6)
    h, c = cell.step(torch.randn(2, 4), LstmState(torch.zeros(2, 6), torch.ones(2, 6)), ctx)       # a 2-tuple to the cell
    st = LstmState(h, c)
    assert st.hidden is h and st.cell is c and len(st) == 2 and GruConfig is LstmConfig and GruState(h).hidden is h
    bi = BidirectionalRnn(GruCell.new(BE, 4, 3, seed=1), GruCell.new(BE, 4, 3, seed=2))
    xs = torch.randn(5, 2, 4)
    out = bi.forward_directions(xs, ctx)
    assert isinstance(out, BidirectionalOutput) and torch.equal(out.concatenated, bi.forward_sequence(xs, ctx)[0])
    assert torch.equal(out.concatenated[..., :3], out.forward) and torch.equal(out.concatenated[..., 3:], out.backward)
    rows = MultiReadout.new(BE, ["a", "b"], 4, threshold=0.5).predict_all(torch.randn(3, 4), ctx)
    assert len(rows) == 3 and [p.label for p in rows[0]] == ["a", "b"] and all(p.predicted == (p.probability >= 0.5) for r in rows for p in r)
    assert all(abs(p.probability - torch.sigmoid(torch.tensor(p.logit)).item()) < 1e-6 for r in rows for p in r)
    det = BinaryReadout.new(BE, 4).predict_detailed(torch.randn(3, 4), ctx)
    assert len(det) == 3 and all(d.predicted == (d.probability >= 0.5) for d in det) and ReadoutConfig(8, 3).labels == 3
    r = ExpertChoiceRouter.new(BE, ExpertChoiceConfig(8, 3, 16, tokens_per_expert=2))
    x = torch.randn(6, 8, generator=torch.Generator().manual_seed(3))
    asg = r.assignments(x)
    idx, gate, _ = r.select(x)
    assert asg.num_tokens == 6 and [asg.tokens_of(e) for e in range(3)] == idx.tolist()
    assert asg.assignments[1][0].expert_idx == 1 and asg.assignments[1][0].weight == pytest.approx(float(gate[1, 0]))
    assert sorted(asg.unrouted_tokens() + sorted({t for e in range(3) for t in asg.tokens_of(e)})) == list(range(6))
    assert all(e in range(3) for e in asg.experts_of(asg.tokens_of(0)[0]))
    layer = SharedExpertLayer.new(BE, SharedExpertConfig(16, 1, 4, 24, top_k=2, shared_weight=0.5, routed_weight=2.0))
    hr = layer.routing(torch.randn(5, 16))
    assert hr.shared_gate.tolist() == [0.5] * 5 and hr.routed_gates.shape == (5, 4) and hr.top_k_indices.shape == (5, 2)
    assert torch.allclose(hr.routed_gates.sum(-1), torch.ones(5), atol=1e-6)
    assert torch.allclose(hr.top_k_weights, 2.0 * hr.routed_gates.gather(1, hr.top_k_indices), atol=1e-6)
    cfg = EncoderDecoderConfig.symmetric(32, 4, 1, 64, dropout=0.0, max_seq_len=16)
    tied = TransformerEncoderDecoder.from_config(BE, cfg, 20, 20)
    untied = TransformerEncoderDecoder.from_config(BE, EncoderDecoderConfig.symmetric(32, 4, 1, 64, dropout=0.0, max_seq_len=16)
                                                   .with_shared_embeddings(False), 20, 20)
    assert tied.decoder.token_embedding is tied.encoder.token_embedding and len(untied.parameters()) == len(tied.parameters()) + 1
    assert len(tied.named_parameters()) == len(untied.named_parameters())      # both names stay in the checkpoint
    y = tied.forward((torch.tensor([[1, 2, 3]]), torch.tensor([[4, 5]])), ForwardCtx.train(BE))
    y.sum().backward()
    g = tied.encoder.token_embedding.embed.tensor.grad
    assert g[[1, 2, 3]].abs().sum() > 0 and g[[4, 5]].abs().sum() > 0          # both uses reach the one table
    from rustral_b200.optim import Sgd
    before = tied.encoder.token_embedding.embed.tensor.detach().clone()
    Sgd(1.0).step(tied.parameters())
    assert torch.allclose(tied.encoder.token_embedding.embed.tensor.detach(), before - g, atol=1e-6)    # stepped once, not twice


def test_quantization_stats_account_for_payload_and_scales():
    from rustral_b200.nn import LinearBuilder, QuantizationScheme, Sequential, quantize_model_with_stats
    model = Sequential(LinearBuilder(128, 64).with_bias().build(BE), LinearBuilder(64, 32).build(BE))
    st = quantize_model_with_stats(model, QuantizationScheme.INT8_PER_CHANNEL)
    weights = 128 * 64 + 64 * 32
    assert st.layers_quantized == 2 and st.scheme is QuantizationScheme.INT8_PER_CHANNEL
    assert st.original_size_mb == pytest.approx(weights * 4 / 2 ** 20)
    assert st.quantized_size_mb == pytest.approx((weights + (64 + 32) * 8) / 2 ** 20)      # int8 payload + fp32 scale and zero point per channel
    assert 3.5 < st.compression_ratio < 4.0
    m4 = Sequential(LinearBuilder(128, 64).build(BE))
    s4 = quantize_model_with_stats(m4, QuantizationScheme.INT4, group_size=64)
    assert s4.quantized_size_mb == pytest.approx((128 * 64 // 2 + 64 * 2 * 4) / 2 ** 20) and s4.compression_ratio > 6.5


def test_distributed_records():
    from rustral_b200.optim import Adam
    from rustral_b200.parallel.checkpoint import DistributedCheckpointManager, ShardData
    from rustral_b200.parallel.fsdp import FSDP, FSDPMemoryStats
    from rustral_b200.parallel.nccl import NcclDataType, NcclRedOp, NcclUniqueId
    from rustral_b200.parallel.pipeline_parallel import PipelineLayer, PipelineSchedule, PipelineStats, pipeline_bubble_fraction
    from rustral_b200.parallel.process_group import CommunicationBackend, ProcessGroup
    from rustral_b200.parallel.zero import ZeroCheckpoint, ZeroOptimizer, ZeRoMemoryStats
    from rustral_b200.parallel.zero_infinity import ZeroInfinityConfig, ZeROInfinityEstimator
    from rustral_b200.nn import LinearBuilder, Sequential
    z1, z2 = ZeRoMemoryStats.zero1(1 << 20, 4, 4), ZeRoMemoryStats.zero2(1 << 20, 4, 4)
    assert (z1.total_params_mb, z1.local_params_mb, z1.local_optimizer_states_mb, z1.local_gradients_mb) == (4.0, 1.0, 2.0, 4.0)
    assert z1.memory_saved_percent == pytest.approx(56.25) and z2.local_gradients_mb == 1.0 and z2.memory_saved_percent == pytest.approx(75.0)
    pg = ProcessGroup.new_single_process()
    assert pg.communication_backend is CommunicationBackend.SINGLE_PROCESS
    assert ProcessGroup.new_threaded(2)[1].communication_backend is CommunicationBackend.THREADED
    lin = LinearBuilder(4, 4).with_bias().build(BE)
    opt = ZeroOptimizer(lin.named_parameters(), pg, lr=0.1)
    lin(torch.ones(1, 4)).sum().backward()
    opt.step()
    ck = ZeroCheckpoint.of(opt)
    assert (ck.rank, ck.world_size) == (0, 1) and ck.inner["t"] == 1
    opt2 = ZeroOptimizer(lin.named_parameters(), pg, lr=0.5)
    ck.restore(opt2)
    assert opt2.t == 1 and opt2.lr == 0.1 and torch.equal(opt2.m, opt.m)
    f = FSDP(Sequential(LinearBuilder(4, 4).build(BE)), Adam(1e-2), pg)
    ms = f.memory_stats()
    assert isinstance(ms, FSDPMemoryStats) and ms.world_size == 1 and ms.total_parameters == 16 and ms.local_parameters == 16
    assert ms.memory_reduction_percent == 0.0 and ms["full_bytes"] == 64 and ms["savings"] == 0.0
    est = ZeROInfinityEstimator.estimate_for(1000, 2, ZeroInfinityConfig(cpu_offload=True, nvme_offload=True))
    assert (est.model_memory, est.optimizer_states, est.gpu_memory, est.cpu_memory, est.nvme_memory, est.total_memory) == (2000, 4000, 4000, 4000, 4000, 12000)
    assert ZeROInfinityEstimator.estimate_for(1000, 2, ZeroInfinityConfig(cpu_offload=False)).total_memory == 4000
    assert NcclDataType.of(torch.bfloat16) is NcclDataType.BFLOAT16 and int(NcclDataType.FLOAT32) == 7 and NcclDataType.FLOAT16.size_bytes() == 2
    assert int(NcclRedOp.AVG) == 4 and NcclRedOp.MAX.op_name == "max"

    class Store(dict):
        def set(self, k, v): self[k] = v
        def get(self, k): return self[k].encode()
    s = Store()
    uid = NcclUniqueId.create(s)
    assert NcclUniqueId.fetch(s) == uid and len(uid.internal) == 128 and NcclUniqueId.create() != uid
    assert PipelineLayer.check(lin) and not PipelineLayer.check(object())
    b = pipeline_bubble_fraction(PipelineSchedule.INTERLEAVED, 4, 8)
    st = PipelineStats(4, 8, "INTERLEAVED", b, 1 - b)
    assert st["bubble_fraction"] == pytest.approx(3 / 11) and st.efficiency == pytest.approx(8 / 11)
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        mgr = DistributedCheckpointManager(pg, d)
        mgr.save(0, 3, [("w", lin.weight)], {"lr": 0.1})
        shard = mgr.load_shard(0)
        assert isinstance(shard, ShardData) and torch.equal(shard.params["w"], lin.weight.tensor.detach()) and shard.optimizer == {"lr": 0.1}


def test_runtime_data_autograd_and_error_types(tmp_path, monkeypatch):
    from rustral_b200.autograd import CheckpointedSegment, GradExt, GradExtFromStore, Tape
    from rustral_b200.data import WikiText2Splits, load_wikitext2_splits
    from rustral_b200.runtime.inference import InferencePool, InferenceResponse
    from rustral_b200.runtime.tape_trainer import Classification, Regression, Trainer
    from rustral_b200.optim import Sgd
    from rustral_b200.symbolic import SymbolicError, Vocabulary
    from rustral_b200.utils import onnx_export
    from rustral_b200.utils.hf import HfError, download_state_dict
    assert Trainer.for_task(Classification, Sgd(0.1))._cls and not Trainer.for_task(Regression, Sgd(0.1))._cls
    with pytest.raises(ValueError):
        Trainer.for_task(int, Sgd(0.1))
    pool = InferencePool(2, 4, lambda x: 1 / x)
    reqs = [pool.submit(v) for v in (1, 2, 0)]
    out = [r.wait(5) for r in reqs]
    assert [o.output for o in out[:2]] == [1.0, 0.5] and isinstance(out[2], InferenceResponse) and isinstance(out[2].error, ZeroDivisionError)
    assert reqs[0].done() and reqs[0].input == 1
    with pytest.raises(ZeroDivisionError):
        out[2].unwrap()
    pool.shutdown()
    d = tmp_path / "datasets" / "wikitext-2"
    d.mkdir(parents=True)
    for s in ("train", "valid", "test"):
        (d / f"{s}.txt").write_text(f"{s} text")
    monkeypatch.setenv("RUSTRAL_CACHE_DIR", str(tmp_path))
    monkeypatch.setenv("RUSTRAL_DATASET_OFFLINE", "1")
    sp = load_wikitext2_splits()
    assert isinstance(sp, WikiText2Splits) and tuple(sp) == ("train text", "valid text", "test text")
    with pytest.raises(HfError) as e:
        download_state_dict("nobody/nothing")                       # offline and not cached
    assert e.value.kind == "hub" and "nobody/nothing" in str(e.value)
    seg = CheckpointedSegment(torch.tensor([1.0, 2.0]), lambda x: x * 3)
    assert seg.recompute().tolist() == [3.0, 6.0] and seg.saved_bytes() == 8 and seg.input_id is None
    p = BE.constant_parameter("p", (2,), 2.0)
    tape = Tape(ForwardCtx.train(BE))
    loss = tape.sum_all_tape(tape.mul(tape.watch_parameter(p), tape.watch_parameter(p)))
    grads = tape.backward(loss)
    assert GradExtFromStore.gradient_from_store(p, grads, tape.param_map).tolist() == [4.0, 4.0]
    assert GradExt.gradient(p, tape).tolist() == [4.0, 4.0]
    v = Vocabulary()
    v.try_insert("a"); v.freeze()
    assert v.try_insert("a") == 1
    with pytest.raises(SymbolicError) as e:
        v.try_insert("b")
    assert e.value.kind == "frozen" and v.insert("b") == 0             # the lenient insert maps to <unk>
    with pytest.raises(SymbolicError) as e:
        v.token_strict(7)
    assert e.value.kind == "id_out_of_range" and v.token_strict(1) == "a"
    with pytest.raises(onnx_export.OnnxExportError) as e:
        onnx_export.export_linear_f32(4, 3, torch.zeros(3, 4), torch.zeros(5))
    assert (e.value.kind, e.value.expected, e.value.got) == ("bias_len", 3, 5)
