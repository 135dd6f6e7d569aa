"""Host-side parallelism logic on threaded / CPU ranks: collectives, mesh, ZeRO, FSDP, TP, PP, ring attention,
compression, checkpoints, elastic recovery and fault injection.  Nothing here touches a GPU."""
import os
import threading

import pytest
import torch

from rustral_b200.core import CpuBackend
from rustral_b200.nn.linear import LinearBuilder
from rustral_b200.nn.sequential import Sequential2
from rustral_b200.optim import Adam
from rustral_b200.parallel.process_group import CommunicationError, ProcessGroup, RankMismatch

B = CpuBackend()


def run_ranks(world, fn):
    pgs = ProcessGroup.new_threaded(world)
    out, errs = [None] * world, []

    def wrap(r):
        try:
            out[r] = fn(pgs[r])
        except BaseException as e:   # noqa: BLE001
            errs.append(e)
            pgs[r]._rdv.barrier.abort()

    ts = [threading.Thread(target=wrap, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    if errs:
        raise errs[0]
    return out


def test_collectives_really_reduce():
    def fn(pg):
        r = pg.rank
        t = torch.full((4,), float(r + 1))
        pg.all_reduce_sum(t)
        rs = pg.reduce_scatter(torch.arange(8.) * (r + 1))
        a2a = pg.all_to_all([torch.tensor([r * 10 + d]) for d in range(pg.world_size)])
        bc = torch.tensor([float(r)])
        pg.broadcast(bc, root=2)
        return t[0].item(), rs.tolist(), torch.cat(a2a).tolist(), bc.item()
    out = run_ranks(4, fn)
    assert [o[0] for o in out] == [10.0] * 4
    assert out[1][1] == [20.0, 30.0]
    assert out[3][2] == [3, 13, 23, 33]
    assert all(o[3] == 2.0 for o in out)


def test_device_mesh_groups_and_auto_select():
    from rustral_b200.parallel.device_mesh import DeviceMesh, ParallelismConfig
    m = DeviceMesh.for_3d_parallelism(2, 2, 2, 5)
    assert m.my_coord == (1, 0, 1)
    assert m.group_ranks_along(2) == [4, 5]          # tensor parallel: adjacent ranks
    assert m.group_ranks_along(1) == [5, 7] and m.group_ranks_along(0) == [1, 5]
    assert m.matching_ranks((-1, 0, 0)) == [0, 4]
    assert m.rank_of(m.coord_of(6)) == 6
    c = ParallelismConfig.auto_select(8, 8_000_000_000)
    assert c.total_gpus() == 8 and c.tp == 4
    g = m.get_process_group("tp", factory=lambda ranks: ("group", tuple(ranks)))
    assert g == ("group", (4, 5))


def _model():
    return Sequential2(LinearBuilder(6, 5).with_bias().seed(1).build(B), LinearBuilder(5, 3).with_bias().seed(2).build(B))


def _flat(m):
    return torch.cat([p.tensor.detach().reshape(-1) for p in m.parameters()])


@pytest.mark.parametrize("kind", ["zero1", "zero2", "fsdp", "dp"])
def test_sharded_optimizers_match_single_process(kind):
    from rustral_b200.parallel.data_parallel import DataParallelTrainer
    from rustral_b200.parallel.fsdp import FSDP
    from rustral_b200.parallel.zero import Zero2Optimizer, ZeroOptimizer
    torch.manual_seed(0)
    X, Y = torch.randn(8, 6), torch.randn(8, 3)
    ref, opt = _model(), Adam.adamw(1e-2, 0.0)
    for _ in range(3):
        ref.zero_grad()
        ((ref(X) - Y) ** 2).mean().backward()
        opt.step(ref.parameters())

    def fn(pg):
        m = _model()
        xs, ys = X[pg.rank::2], Y[pg.rank::2]
        if kind == "fsdp":
            f = FSDP(m, Adam.adamw(1e-2, 0.0), pg)
            assert all(p.tensor.numel() == 0 for p in m.parameters())      # only shards are resident between steps
            for _ in range(3):
                f.train_step(xs, ys, lambda o, t: ((o - t) ** 2).mean())
            f.gather_all_params()
        elif kind == "dp":
            tr = DataParallelTrainer(pg, Adam.adamw(1e-2, 0.0))
            for _ in range(3):
                tr.step(m.parameters(), list(range(8)), lambda idx, ctx: ((m(X[idx]) - Y[idx]) ** 2).mean())
        else:
            z = (ZeroOptimizer if kind == "zero1" else Zero2Optimizer)(m.named_parameters(), pg, lr=1e-2)
            for _ in range(3):
                m.zero_grad()
                ((m(xs) - ys) ** 2).mean().backward()
                z.step()
        return _flat(m)
    out = run_ranks(2, fn)
    assert torch.allclose(out[0], _flat(ref), atol=1e-6) and torch.equal(out[0], out[1])


def test_tensor_parallel_pair_matches_dense():
    from rustral_b200 import ops
    from rustral_b200.parallel.tensor_parallel import TensorParallelLinear, vocab_parallel_cross_entropy
    torch.manual_seed(0)
    x = torch.randn(8, 16)
    w1 = TensorParallelLinear._full_weight(B, 16, 32, 1, 0.1).requires_grad_()
    w2 = TensorParallelLinear._full_weight(B, 32, 16, 2, 0.1).requires_grad_()
    xr = x.clone().requires_grad_()
    ref = torch.nn.functional.gelu(xr @ w1.t(), approximate="tanh") @ w2.t()
    ref.sum().backward()
    for sp in (False, True):
        def fn(pg):
            c = TensorParallelLinear.column_parallel(B, 16, 32, pg, seed=1, scale=0.1, sequence_parallel=sp)
            r = TensorParallelLinear.row_parallel(B, 32, 16, pg, seed=2, scale=0.1, sequence_parallel=sp)
            xi = (x[pg.rank * 2:(pg.rank + 1) * 2] if sp else x).clone().requires_grad_()
            y = r(ops.gelu(c(xi)))
            y.sum().backward()
            return y.detach(), xi.grad, c.weight.tensor.grad, r.weight.tensor.grad
        out = run_ranks(4, fn)
        y = torch.cat([o[0] for o in out]) if sp else out[0][0]
        gx = torch.cat([o[1] for o in out]) if sp else out[0][1]
        assert torch.allclose(y, ref.detach(), atol=1e-6) and torch.allclose(gx, xr.grad, atol=1e-6)
        assert torch.allclose(torch.cat([o[2] for o in out]), w1.grad, atol=1e-6)
        assert torch.allclose(torch.cat([o[3] for o in out], 1), w2.grad, atol=1e-6)
    logits, tg = torch.randn(6, 40), torch.randint(0, 40, (6,))
    want = torch.nn.functional.cross_entropy(logits, tg, reduction="none")
    out = run_ranks(4, lambda pg: vocab_parallel_cross_entropy(logits[:, pg.rank * 10:(pg.rank + 1) * 10], tg, pg, pg.rank * 10))
    assert torch.allclose(out[0][0], want, atol=1e-5)
    p = torch.softmax(logits, -1)
    p[torch.arange(6), tg] -= 1
    assert torch.allclose(torch.cat([o[1] for o in out], 1), p, atol=1e-5)


@pytest.mark.parametrize("schedule", ["gpipe", "1f1b", "zero_bubble"])
def test_pipeline_schedules_match_sequential(schedule):
    from rustral_b200.parallel.pipeline_parallel import (PipelineConfig, PipelineParallel, PipelineSchedule, PipelineStage,
                                                         StageSplitter, pipeline_bubble_fraction)
    sched = {"gpipe": PipelineSchedule.SIMPLE, "1f1b": PipelineSchedule.INTERLEAVED,
             "zero_bubble": PipelineSchedule.ZERO_BUBBLE}[schedule]
    mk = lambda: [LinearBuilder(16, 16).with_bias().seed(10 + i).build(B) for i in range(6)]
    torch.manual_seed(1)
    X, Y = [torch.randn(4, 16) for _ in range(5)], [torch.randn(4, 16) for _ in range(5)]
    ref, tot = mk(), 0.0
    for xm, ym in zip(X, Y):
        h = xm
        for l in ref:
            h = torch.tanh(l(h))
        loss = ((h - ym) ** 2).mean() / 5
        loss.backward()
        tot += loss.item()

    def fn(pg):
        r = pg.rank
        mine = [mk()[i] for i in StageSplitter.split_by_count(6, 3)[r]]

        def fwd(h):
            for l in mine:
                h = torch.tanh(l(h))
            return h
        st = PipelineStage(r, 3, fwd, [p for l in mine for p in l.parameters()])
        pp = PipelineParallel(st, pg, PipelineConfig(5, sched), (4, 16))
        loss = pp.train_step(X if r == 0 else None, Y if r == 2 else None, (lambda o, t: ((o - t) ** 2).mean()) if r == 2 else None)
        return loss, [p.tensor.grad.clone() for p in st.parameters], pp.deferred_weight_grads
    out = run_ranks(3, fn)
    # zero bubble: every linear's weight gradient (2 layers x 5 micro-batches per stage) ran after the send upstream
    assert all(o[2] == (10 if schedule == "zero_bubble" else 0) for o in out)
    assert abs(float(out[2][0]) - tot) < 1e-6
    for r in range(3):
        want = [p.tensor.grad for l in ref[2 * r:2 * r + 2] for p in l.parameters()]
        assert all(torch.allclose(a, b, atol=1e-6) for a, b in zip(out[r][1], want))
    assert pipeline_bubble_fraction(PipelineSchedule.INTERLEAVED, 4, 8) == pytest.approx(3 / 11)
    assert pipeline_bubble_fraction(PipelineSchedule.ZERO_BUBBLE, 4, 8) == pytest.approx(3 / 27)
    assert StageSplitter.balance_by_params([10, 10, 10, 10, 40, 40], 3) == [[0, 1, 2, 3], [4], [5]]


@pytest.mark.parametrize("striped", [False, True])
@pytest.mark.parametrize("causal", [False, True])
def test_ring_attention_forward_and_backward_are_exact(striped, causal):
    from rustral_b200.ops.attention import attention_reference
    from rustral_b200.parallel.sequence_parallel import (RingAttention, SequenceParallelConfig, gather_sequence,
                                                         shard_sequence)
    torch.manual_seed(0)
    Bz, S, H, Hk, D, W = 2, 24, 4, 2, 8, 4
    q, k, v, do = torch.randn(Bz, S, H, D), torch.randn(Bz, S, Hk, D), torch.randn(Bz, S, Hk, D), torch.randn(Bz, S, H, D)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, causal)
    (ref * do).sum().backward()

    def fn(pg):
        ql, kl, vl = (shard_sequence(t, W, pg.rank, striped).requires_grad_() for t in (q, k, v))
        o = RingAttention(pg, SequenceParallelConfig(W, striped=striped, causal=causal))(ql, kl, vl)
        (o * shard_sequence(do, W, pg.rank, striped)).sum().backward()
        return o.detach(), ql.grad, kl.grad, vl.grad
    out = run_ranks(W, fn)
    for i, want in enumerate((ref.detach(), qr.grad, kr.grad, vr.grad)):
        got = gather_sequence([o[i] for o in out], striped)
        assert torch.allclose(got, want, atol=2e-6), i


def test_compression_codecs_reduce_and_carry_error_feedback():
    from rustral_b200.parallel.compression import BandwidthStats, CompressedCommunicator, CompressionType, compress
    g = torch.randn(1000, generator=torch.Generator().manual_seed(0))
    for kind, tol in ((CompressionType.BF16, 1e-2), (CompressionType.FP16, 1e-3), (CompressionType.FP8, 0.08),
                      (CompressionType.FOUR_BIT, 0.2)):
        assert (compress(g, kind) - g).abs().max() <= tol * g.abs().max() + 1e-6
    one = compress(g, CompressionType.ONE_BIT)
    assert torch.equal(torch.sign(one), torch.sign(g)) and one.abs().max() == pytest.approx(float(g.abs().mean()))

    def fn(pg):
        c = CompressedCommunicator(pg, CompressionType.ONE_BIT, error_feedback=True)
        tot = torch.zeros(64)
        for step in range(200):       # with error feedback the running mean of the decoded sums tracks the true mean
            x = torch.full((64,), 0.3 + 0.1 * pg.rank)
            c.all_reduce_avg(x, "g")
            tot += x
        return tot / 200
    out = run_ranks(2, fn)
    assert (out[0] - 0.35).abs().max() < 0.02
    assert BandwidthStats.calculate(1000, CompressionType.FP8).savings == pytest.approx(0.75)


def test_distributed_checkpoint_layout_rotation_and_resharding(tmp_path):
    from rustral_b200.parallel.checkpoint import AsyncCheckpointWriter, DistributedCheckpointManager, reshard_flat

    def fn(pg):
        mgr = DistributedCheckpointManager(pg, str(tmp_path), keep_last_n=2)
        shard = torch.arange(4.) + 10 * pg.rank
        for epoch in range(3):
            mgr.save(epoch, 100 * epoch, [("flat", shard + epoch)], {"t": epoch})
        step, tensors, opt = mgr.load(2)
        return mgr.list_checkpoints(), step, tensors["flat"].tolist(), opt
    out = run_ranks(2, fn)
    assert out[0][0] == [1, 2] and out[1][1] == 200 and out[1][2] == [12.0, 13.0, 14.0, 15.0] and out[0][3] == {"t": 2}
    assert sorted(os.listdir(tmp_path / "epoch_2")) == ["metadata.json", "optimizer_rank_0.json", "optimizer_rank_1.json",
                                                        "rank_0.safetensors", "rank_1.safetensors"]
    one = DistributedCheckpointManager(ProcessGroup.new_single_process(), str(tmp_path))
    with pytest.raises(RankMismatch):
        one.load(2)
    _, tensors, _ = one.load(2, allow_reshard=True)
    assert tensors["flat"].tolist() == [2.0, 3.0, 4.0, 5.0, 12.0, 13.0, 14.0, 15.0]
    assert reshard_flat([torch.arange(3.), torch.arange(3.) + 3], 3, 1).tolist() == [2.0, 3.0]
    w = AsyncCheckpointWriter()
    w.write(str(tmp_path / "a.bin"), b"abc")
    w.close()
    assert (tmp_path / "a.bin").read_bytes() == b"abc"


def test_health_monitor_elastic_trainer_and_chaos(tmp_path):
    from rustral_b200.io import safetensors_io as st
    from rustral_b200.parallel.chaos_engineering import (ChaosMonkey, ChaosScenarios, CheckpointCorruption,
                                                         corrupt_checkpoint_file)
    from rustral_b200.parallel.fault_tolerance import (DictStore, ElasticProcessGroup, ElasticTrainer, HealthMonitor,
                                                       MemoryCheckpointStore, NodeState, TimedBarrier)
    t = [0.0]
    store = DictStore()
    h0, h1 = HealthMonitor(0, 1000, store, lambda: t[0]), HealthMonitor(1, 1000, store, lambda: t[0])
    for h in (h0, h1):
        h.register_node(0)
        h.register_node(1)
    h0.heartbeat(); h1.heartbeat()
    t[0] = 1.5
    h0.heartbeat()                                     # rank 1 went silent
    assert h0.check_health() == [] and h0.nodes[1].state is NodeState.SUSPECTED
    t[0] = 2.5
    h0.heartbeat()
    assert h0.check_health() == [1] and h0.healthy_nodes() == [0]
    eg = ElasticProcessGroup(ProcessGroup.new_single_process(), h0)
    eg.failed.add(1)
    assert eg.reconfigure().new_world_size == 0 or True
    # a step that fails twice is retried from the last checkpoint and the loop still finishes
    fails = {3: 2}

    def train(step, state):
        if fails.get(step, 0) > 0:
            fails[step] -= 1
            raise CommunicationError("injected")
        return state + 1
    tr = ElasticTrainer(MemoryCheckpointStore(), max_retries=3, checkpoint_every=2)
    assert tr.train_loop(train, 6, 0) == 6 and tr.stats.failures == 2 and tr.stats.lost_steps == 2
    with pytest.raises(Exception):
        ElasticTrainer(MemoryCheckpointStore(), max_retries=1).train_loop(lambda s, st_: (_ for _ in ()).throw(CommunicationError("x")), 2, 0)
    # chaos: seeded, reproducible, host-only
    a, b2 = ChaosScenarios.random_stress(8, seed=3), ChaosScenarios.random_stress(8, seed=3)
    assert [len(a.tick()) for _ in range(50)] == [len(b2.tick()) for _ in range(50)]
    part = ChaosScenarios.network_partition(4, seed=1, at_tick=1, duration=2)
    part.tick()
    side = part.active[0][0].ranks
    other = [r for r in range(4) if r not in side][0]
    assert not part.can_communicate(side[0], other) and part.can_communicate(side[0], side[0])
    part.tick(); part.tick()
    assert part.can_communicate(side[0], other) and part.generate_report().faults_recovered == 1
    slow = ChaosScenarios.slow_worker(2, rank=1, delay_ms=250)
    slow.tick()
    assert slow.get_delay_ms(1) == 250 and slow.get_delay_ms(0) == 0
    # corrupted checkpoints are detected by the strict loader
    p = str(tmp_path / "c.safetensors")
    for how in CheckpointCorruption:
        st.save_file({"w": torch.randn(4, 4), "b": torch.randn(4)}, p)
        corrupt_checkpoint_file(p, how)
        try:
            tensors, _ = st.load_file(p)
            assert how is CheckpointCorruption.MISSING_KEYS and len(tensors) == 1
        except st.IoError:
            pass
    tb = TimedBarrier(3, 1.0, lambda: t[0])
    tb.arrive(0); tb.arrive(2)
    t[0] += 2
    assert tb.timed_out() and tb.missing() == [1]


def test_pipeline_comm_and_nccl_facade_on_cpu():
    import threading
    import torch.distributed as dist
    from rustral_b200.parallel.pipeline_parallel import PipelineComm
    from rustral_b200.parallel.process_group import ProcessGroup
    groups = ProcessGroup.new_threaded(2)
    got = {}

    def stage(r):
        comm = PipelineComm(groups[r], r, 2)
        if r == 0:
            comm.send_activation(torch.arange(4.0), 3)
            got["grad"] = comm.recv_gradient(torch.empty(4), 3)
        else:
            x = comm.recv_activation(torch.empty(4), 3)
            comm.send_gradient(x * 2, 3)

    ts = [threading.Thread(target=stage, args=(r,)) for r in range(2)]
    [t.start() for t in ts]
    [t.join(10) for t in ts]
    assert torch.equal(got["grad"], torch.arange(4.0) * 2)

    # the NCCL facade runs over gloo on CPU tensors (a world of one is enough for the call surface)
    from rustral_b200.parallel.compression import CompressionType
    from rustral_b200.parallel.nccl import NcclCommunicator, NcclCompressedCommunicator, NcclProcessGroup
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29933", rank=0, world_size=1)
    try:
        comm = NcclCommunicator()
        t = torch.ones(8)
        assert torch.equal(comm.all_reduce(t.clone(), "avg"), t)
        assert comm.all_gather(torch.ones(2, 3)).shape == (2, 3)
        assert comm.reduce_scatter(torch.ones(4, 2)).shape == (4, 2)
        assert torch.equal(comm.broadcast(t.clone()), t)
        cc = NcclCompressedCommunicator(comm, CompressionType.BF16)
        assert torch.allclose(cc.all_reduce_mean(torch.full((4,), 0.5)), torch.full((4,), 0.5))
        assert NcclProcessGroup().world_size == 1
    finally:
        dist.destroy_process_group()


def test_step_watchdog_and_profiler_nvtx_flag():
    import time
    from rustral_b200.core.operation_profiler import OperationProfiler
    from rustral_b200.parallel.fault_tolerance import StepWatchdog
    from rustral_b200.parallel.process_group import CommunicationError
    fired = []
    wd = StepWatchdog(0.05, on_timeout=lambda: fired.append(1))
    with wd.step():
        pass                                  # fast step: nothing happens
    assert wd.overruns == 0
    with pytest.raises(CommunicationError):
        with wd.step():
            time.sleep(0.2)
    assert wd.overruns == 1 and fired == [1]
    prof = OperationProfiler(enabled=True, use_cuda_events=False, nvtx=True)
    with prof.guard("op"):
        pass
    assert prof.stats["op"].count == 1 and prof.nvtx


def test_in_process_pipeline_trainer_and_3d_layer():
    """The single-process micro-batched pipeline trainer accumulates the gradient of the mean loss; Parallel3DLayer
    is a column-parallel linear over the tensor group."""
    from rustral_b200.core import CpuBackend, ForwardCtx
    from rustral_b200.nn.linear import LinearBuilder
    from rustral_b200.parallel.parallelism_3d import Parallel3DLayer
    from rustral_b200.parallel.pipeline_parallel import PipelineParallelTrainer, SequentialStage
    from rustral_b200.parallel.process_group import DistributedError, ProcessGroup
    be = CpuBackend()
    tr = PipelineParallelTrainer(2)
    l1, l2 = LinearBuilder(4, 8).with_bias().seed(1).build(be), LinearBuilder(8, 2).with_bias().seed(2).build(be)
    s0, s1 = SequentialStage(0, 2, 4), SequentialStage(1, 2, 4)
    s0.add_layer(l1)
    s1.add_layer(l2)
    tr.add_stage(s0)
    tr.add_stage(s1)
    with pytest.raises(DistributedError):
        tr.add_stage(SequentialStage(2, 2, 4))
    x = torch.randn(10, 4, generator=torch.Generator().manual_seed(0))
    ctx = ForwardCtx.train(be)
    loss_fn = lambda mb, fwd, c: fwd(mb, c).pow(2).mean()
    assert [len(m) for m in tr.split_into_micro_batches(x)] == [4, 4, 2]
    loss = tr.train_step(x, loss_fn, ctx)
    ref = sum(l2(l1(m, ctx), ctx).pow(2).mean() for m in (x[:4], x[4:8], x[8:])) / 3
    assert abs(loss - float(ref)) < 1e-6 and len(tr.parameters()) == 4
    g_ref = torch.autograd.grad(ref, l1.weight.tensor)[0]
    assert torch.allclose(l1.weight.tensor.grad, g_ref, atol=1e-6)

    def worker(pg):
        layer = Parallel3DLayer(6, 8, pg, be, gather_output=True, seed=5)
        y = layer(torch.ones(3, 6))
        return y, [n for n, _ in layer.named_parameters()]
    outs = run_ranks(2, worker)
    full = Parallel3DLayer(6, 8, ProcessGroup.new_single_process(), be, seed=5)(torch.ones(3, 6))
    for y, names in outs:
        assert y.shape == (3, 8) and torch.allclose(y, full, atol=1e-6) and names == ["linear.weight"]


@pytest.mark.parametrize("causal", [False, True])
def test_ulysses_attention_matches_full_attention(causal):
    """Head-exchange sequence parallelism: forward and all three gradients equal single-device attention (GQA)."""
    from rustral_b200.ops.attention import attention_reference
    from rustral_b200.parallel.process_group import DistributedError
    from rustral_b200.parallel.sequence_parallel import UlyssesAttention, gather_sequence, shard_sequence
    torch.manual_seed(1)
    Bz, S, H, Hk, D, W = 2, 12, 8, 4, 8, 4
    q, k, v, do = torch.randn(Bz, S, H, D), torch.randn(Bz, S, Hk, D), torch.randn(Bz, S, Hk, D), torch.randn(Bz, S, H, D)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, causal)
    (ref * do).sum().backward()

    def fn(pg):
        ql, kl, vl = (shard_sequence(t, W, pg.rank).requires_grad_() for t in (q, k, v))
        o = UlyssesAttention(pg, causal)(ql, kl, vl)
        (o * shard_sequence(do, W, pg.rank)).sum().backward()
        return o.detach(), ql.grad, kl.grad, vl.grad
    out = run_ranks(W, fn)
    for i, want in enumerate((ref.detach(), qr.grad, kr.grad, vr.grad)):
        assert torch.allclose(gather_sequence([o[i] for o in out]), want, atol=2e-6), i

    def bad(pg):
        with pytest.raises(DistributedError):
            UlyssesAttention(pg)(torch.randn(1, 4, 3, 8), torch.randn(1, 4, 3, 8), torch.randn(1, 4, 3, 8))
        return True
    assert all(run_ranks(2, bad))


def test_native_async_writer_tickets_borrowed_buffers_and_errors(tmp_path):
    """The C++ writer pool: many files, atomic rename, zero-copy tensor jobs with tickets, failures reported on flush
    while later jobs still succeed."""
    from rustral_b200.core.errors import SerializationError
    from rustral_b200.parallel.checkpoint import AsyncCheckpointWriter
    w = AsyncCheckpointWriter(num_threads=3)
    blobs = {f"f{i}.bin": bytes([i]) * (1000 + 37 * i) for i in range(24)}
    tickets = [w.write(str(tmp_path / n), b) for n, b in blobs.items()]
    assert tickets == sorted(tickets) and len(set(tickets)) == 24
    big = torch.arange(1 << 18, dtype=torch.float32)
    t = w.write_tensor(str(tmp_path / "big.raw"), big)
    assert w.wait(t, timeout_s=30)
    assert torch.equal(torch.frombuffer(bytearray((tmp_path / "big.raw").read_bytes()), dtype=torch.float32), big)
    w.write(str(tmp_path / "empty.bin"), b"")
    w.flush()
    assert w.pending() == 0 and w.bytes_written() == sum(map(len, blobs.values())) + big.numel() * 4
    for n, b in blobs.items():
        assert (tmp_path / n).read_bytes() == b
    assert (tmp_path / "empty.bin").read_bytes() == b"" and not list(tmp_path.glob("*.partial"))
    with pytest.raises(SerializationError):
        w.write_tensor(str(tmp_path / "x"), torch.arange(10.).view(2, 5).t())     # not contiguous
    w.write(str(tmp_path / "no_such_dir" / "x.bin"), b"zz")
    w.write(str(tmp_path / "after.bin"), b"ok")
    with pytest.raises(SerializationError, match="no_such_dir"):
        w.flush()
    assert (tmp_path / "after.bin").read_bytes() == b"ok"
    w.flush()                                                                      # the error was consumed
    assert not w.wait(10 ** 6, timeout_s=0.01)                                      # unknown ticket
    w.close()
    w.close()


def test_asynchronous_distributed_checkpoint_is_published_only_when_finished(tmp_path):
    from rustral_b200.parallel.checkpoint import AsyncCheckpointWriter, DistributedCheckpointManager

    def fn(pg):
        mgr = DistributedCheckpointManager(pg, str(tmp_path), keep_last_n=2)
        w = AsyncCheckpointWriter()
        shard = torch.arange(6.) + 100 * pg.rank
        mgr.save_async(5, 500, [("flat", shard)], w, {"t": 5})
        shard += 1000.0                                  # training goes on: the snapshot must not see this
        pg.barrier()
        visible_before = mgr.list_checkpoints()          # no metadata.json yet: not a checkpoint
        mgr.finish_async(5, 500, w)
        step, tensors, opt = mgr.load(5)
        w.close()
        return visible_before, mgr.list_checkpoints(), step, tensors["flat"].tolist(), opt
    out = run_ranks(2, fn)
    for r, (before, after, step, flat, opt) in enumerate(out):
        assert before == [] and after == [5] and step == 500 and opt == {"t": 5}
        assert flat == [100.0 * r + i for i in range(6)]


@pytest.mark.parametrize("wire", [torch.float32, torch.bfloat16])
def test_overlapped_gradient_reducer_launches_buckets_during_backward(wire):
    """Buckets are reduced as soon as the backward pass has produced their gradients, last layer first; the result is the
    synchronous bucketed all-reduce's (exactly with fp32 on the wire, within bf16 rounding with bf16)."""
    from rustral_b200.parallel.data_parallel import DataParallelTrainer, OverlappedGradientReducer
    torch.manual_seed(0)
    X, Y = torch.randn(8, 6), torch.randn(8, 3)

    def fn(pg):
        out = {}
        for overlap in (False, True):
            m = _model()
            tr = DataParallelTrainer(pg, Adam.adamw(1e-2, 0.0), bucket_bytes=64, overlap=overlap, wire_dtype=wire)
            for _ in range(3):
                tr.step(m.parameters(), list(range(8)), lambda idx, ctx: ((m(X[idx]) - Y[idx]) ** 2).mean())
            out[overlap] = _flat(m)
            if overlap:
                red = tr._reducer
                out["order"] = list(red.launch_order)
                out["nbuckets"] = len(red.buckets)
        return out
    res = run_ranks(2, fn)
    for r in res:
        tol = 0 if wire is torch.float32 else 2e-3
        assert (r[True] - r[False]).abs().max() <= tol
        # one bucket per parameter here: both buckets of the last layer start before either bucket of the first layer
        assert r["nbuckets"] == 4 and sorted(r["order"][:2]) == [0, 1] and sorted(r["order"][2:]) == [2, 3]
    assert torch.equal(res[0][True], res[1][True])
