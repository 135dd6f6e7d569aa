"""Host-side parallel components one by one: mesh arithmetic, the strategy chooser, gradient-compression codecs with their
error bounds, error feedback, the offloaded optimizer's NVMe spill, and the distributed checkpoint manager
(crates/distributed/src/{device_mesh,compression,zero_infinity,checkpoint}.rs `mod tests`)."""
import math
import os

import pytest
import torch
from hypothesis import given, settings, strategies as hs

from rustral_b200.core import Parameter
from rustral_b200.core.errors import SerializationError
from rustral_b200.parallel.checkpoint import (AsyncCheckpointWriter, DistributedCheckpointManager, ShardedCheckpoint, reshard_flat)
from rustral_b200.parallel.compression import (BandwidthStats, CompressedCommunicator, CompressionType, ErrorFeedbackCompression,
                                               OneBitAdam, compress)
from rustral_b200.parallel.device_mesh import DeviceMesh, ParallelismConfig
from rustral_b200.parallel.process_group import DistributedError, ProcessGroup, RankMismatch
from rustral_b200.parallel.zero_infinity import StorageLocation, ZeroInfinity, ZeroInfinityConfig, ZeROInfinityEstimator


# ---- device mesh ------------------------------------------------------------------------------------------------------
@settings(max_examples=60, deadline=None)
@given(hs.lists(hs.integers(1, 4), min_size=1, max_size=4), hs.data())
def test_mesh_rank_and_coordinate_are_inverse_and_groups_partition_the_world(shape, data):
    world = math.prod(shape)
    rank = data.draw(hs.integers(0, world - 1))
    m = DeviceMesh(shape, rank)
    assert m.rank_of(m.coord_of(rank)) == rank and m.world_size == world
    assert [m.rank_of(m.coord_of(r)) for r in range(world)] == list(range(world))
    for dim in range(len(shape)):
        groups = m.all_groups_along(dim)
        assert sorted(r for g in groups for r in g) == list(range(world))          # disjoint cover
        assert all(len(g) == shape[dim] for g in groups) and rank in m.group_ranks_along(dim)
        mine = m.group_ranks_along(dim)
        assert all(tuple(c for i, c in enumerate(m.coord_of(r)) if i != dim) ==
                   tuple(c for i, c in enumerate(m.my_coord) if i != dim) for r in mine)


def test_mesh_rejects_bad_shapes_ranks_and_patterns():
    with pytest.raises(DistributedError):
        DeviceMesh((2, 0), 0)
    with pytest.raises(DistributedError):
        DeviceMesh((2, 2), 4)
    m = DeviceMesh((2, 3), 0, ("a", "b"))
    with pytest.raises(DistributedError):
        m.rank_of((0, 3))
    with pytest.raises(DistributedError):
        m.matching_ranks((0,))
    assert m.matching_ranks((-1, 1)) == [1, 4] and m.matching_ranks((1, -1)) == [3, 4, 5] and m.dim_names == ("a", "b")


def test_3d_mesh_puts_tensor_parallel_ranks_next_to_each_other():
    m = DeviceMesh.for_3d_parallelism(2, 4, 2, rank=5)
    tp = m.group_ranks_along(m.dim_names.index("tp"))
    assert tp == [4, 5, 6, 7] and len(m.group_ranks_along(m.dim_names.index("dp"))) == 2
    assert len(m.group_ranks_along(m.dim_names.index("pp"))) == 2 and m.world_size == 16


@pytest.mark.parametrize("gpus,params,want", [(8, 100_000_000, (8, 1, 1)), (8, 2_000_000_000, (2, 4, 1)),
                                              (64, 20_000_000_000, (2, 8, 4)), (1, 50_000_000_000, (1, 1, 1)),
                                              (6, 5_000_000_000, (2, 3, 1))])
def test_auto_select_thresholds(gpus, params, want):
    c = ParallelismConfig.auto_select(gpus, params)
    assert (c.dp, c.tp, c.pp) == want and c.total_gpus() == gpus


# ---- compression ----------------------------------------------------------------------------------------------------
def _vec(n=4096, seed=0):
    return torch.randn(n, generator=torch.Generator().manual_seed(seed))


@pytest.mark.parametrize("kind,rel", [(CompressionType.NONE, 0.0), (CompressionType.FP16, 2 ** -11), (CompressionType.BF16, 2 ** -8),
                                      (CompressionType.FP8, 2 ** -4)])
def test_float_codecs_stay_within_half_an_ulp_of_their_format(kind, rel):
    x = _vec()
    y = compress(x, kind)
    big = x.abs() > 0.05 * x.abs().max()           # below that fp8 runs into its subnormals
    assert float(((y - x).abs() / x.abs())[big].max()) <= rel + 1e-9


def test_four_bit_error_is_bounded_by_half_a_step_of_its_group_and_one_bit_keeps_sign_and_l1():
    x = _vec(1000, 1)                              # not a multiple of the group: the tail is padded
    y = compress(x, CompressionType.FOUR_BIT, group=64)
    assert y.shape == x.shape
    for g0 in range(0, 1000, 64):
        xs, ys = x[g0:g0 + 64], y[g0:g0 + 64]
        assert float((xs - ys).abs().max()) <= float(xs.abs().max()) / 14.0 + 1e-6
    z = compress(x, CompressionType.ONE_BIT)
    assert torch.equal(torch.sign(z), torch.sign(x)) and float(z.abs().sum()) == pytest.approx(float(x.abs().sum()), rel=1e-5)


def test_error_feedback_makes_the_running_sum_track_the_true_sum():
    """Without the residual a 1-bit codec's error accumulates; with it the sum of decoded messages stays within one
    message's error of the sum of inputs."""
    ef = ErrorFeedbackCompression(CompressionType.ONE_BIT)
    true = torch.zeros(256)
    sent = torch.zeros(256)
    plain = torch.zeros(256)
    for s in range(200):
        g = _vec(256, 100 + s) * 0.1 + 0.05
        true += g
        sent += ef.compress(g)
        plain += compress(g, CompressionType.ONE_BIT)
    assert torch.allclose(true - sent, ef.residual, atol=1e-4)
    assert float((true - sent).abs().max()) < 0.25 * float((true - plain).abs().max())


def test_compressed_all_reduce_counts_bytes_and_keeps_one_residual_per_name():
    pg = ProcessGroup.new_single_process()
    comm = CompressedCommunicator(pg, CompressionType.FP8, error_feedback=True)
    a, b = _vec(512, 3), _vec(128, 4)
    a0 = a.clone()
    comm.all_reduce_sum(a, "a")
    comm.all_reduce_avg(b, "b")
    assert comm.bytes_sent == 512 + 128 and comm.bytes_uncompressed == 4 * (512 + 128)
    assert set(comm.residual) == {"a", "b"} and torch.allclose(comm.residual["a"], a0 - a, atol=1e-6)
    st = BandwidthStats.calculate(1000, CompressionType.FOUR_BIT)
    assert (st.uncompressed_bytes, st.compressed_bytes) == (4000, 500) and st.savings == pytest.approx(0.875)
    assert CompressionType.ONE_BIT.ratio == 32.0


def test_one_bit_adam_switches_codec_after_warmup():
    from rustral_b200.optim import Adam
    pg = ProcessGroup.new_single_process()
    p = Parameter("w", torch.zeros(16))
    opt = OneBitAdam(Adam(0.1), pg, warmup_steps=2)
    grads = []
    for s in range(3):
        p.tensor.grad = _vec(16, 20 + s)
        g0 = p.tensor.grad.clone()
        opt.step([p])
        grads.append((g0, p.tensor.grad.clone()))
    assert torch.equal(grads[0][0], grads[0][1]) and torch.equal(grads[1][0], grads[1][1])       # warm-up: exact
    assert len(torch.unique(grads[2][1].abs())) == 1 and opt.comm.bytes_sent == 2                # then sign * magnitude


# ---- offloaded optimizer --------------------------------------------------------------------------------------------
def test_zero_infinity_matches_adamw_and_survives_an_nvme_round_trip(tmp_path):
    from rustral_b200.optim import AdamW
    cfg = ZeroInfinityConfig(nvme_offload=True, nvme_path=str(tmp_path / "spill.bin"), pin_memory=False)
    a, b = Parameter("a", _vec(300, 5)), Parameter("b", _vec(50, 6))
    ra, rb = Parameter("a", a.tensor.clone()), Parameter("b", b.tensor.clone())
    zi = ZeroInfinity(cfg, lr=0.01, weight_decay=0.1)
    zi.register_parameters([a, b])
    ref = AdamW(0.01, weight_decay=0.1)
    for s in range(4):
        for p, r in ((a, ra), (b, rb)):
            g = _vec(p.numel(), 30 + s)
            p.tensor.grad = g.clone()
            r.tensor.grad = g.clone()
        zi.step([a, b])
        ref.step([ra, rb])
        assert all(st.location == StorageLocation.NVME and st.m is None for st in zi.states.values())
    assert torch.allclose(a.tensor, ra.tensor, atol=1e-6) and torch.allclose(b.tensor, rb.tensor, atol=1e-6)
    assert zi.memory_stats() == {"host_bytes": 0, "nvme_bytes": 12 * 350, "gpu_bytes": 0}
    assert os.path.getsize(cfg.nvme_path) == 12 * 350                                   # slots are reused, not appended
    zi.load_from_nvme(a.id)
    assert zi.states[a.id].location == StorageLocation.CPU and zi.memory_stats()["host_bytes"] == 12 * 300


def test_zero_infinity_enforces_its_nvme_quota_and_estimates_memory(tmp_path):
    cfg = ZeroInfinityConfig(nvme_offload=True, nvme_path=str(tmp_path / "s.bin"), nvme_quota=1000, pin_memory=False)
    p = Parameter("p", torch.zeros(100))
    zi = ZeroInfinity(cfg)
    zi.register_parameters([p])
    with pytest.raises(RuntimeError, match="quota"):
        zi.save_to_nvme(p.id)
    est = ZeROInfinityEstimator.estimate(1_000_000, world=4)
    assert est == {"gpu_bytes": 6_000_000, "host_bytes": 3_000_000}


# ---- checkpoints ----------------------------------------------------------------------------------------------------
def test_checkpoint_manager_round_trip_rotation_and_incomplete_epochs(tmp_path):
    pg = ProcessGroup.new_single_process()
    mgr = DistributedCheckpointManager(pg, str(tmp_path), keep_last_n=2)
    w = Parameter("w", _vec(10, 7))
    for e in range(4):
        w.tensor.data.fill_(float(e))
        mgr.save(e, 10 * e, [("w", w)], {"lr": 0.1 * e})
    assert mgr.list_checkpoints() == [2, 3] and mgr.latest_checkpoint() == 3 and not os.path.exists(tmp_path / "epoch_0")
    os.makedirs(tmp_path / "epoch_9")                         # a crash before metadata.json: not a checkpoint
    assert mgr.latest_checkpoint() == 3
    dst = Parameter("w", torch.zeros(10))
    step, tensors, opt = mgr.load(2, [("w", dst)])
    assert step == 20 and opt == {"lr": 0.2} and torch.equal(dst.tensor, torch.full((10,), 2.0))
    assert mgr.read_metadata(3).world_size == 1
    with pytest.raises(SerializationError):
        mgr.load(3, [("missing", dst)])
    with pytest.raises(SerializationError):
        mgr.load(3, [("w", Parameter("w", torch.zeros(11)))])
    with pytest.raises(SerializationError):
        mgr.read_metadata(9)


def test_checkpoint_from_another_world_size_needs_reshard_permission(tmp_path):
    pgs = ProcessGroup.new_threaded(2)
    import threading
    full = torch.arange(10.0)

    def save(rank):
        DistributedCheckpointManager(pgs[rank], str(tmp_path)).save(0, 5, [("flat", full[rank * 5:(rank + 1) * 5])])
    ts = [threading.Thread(target=save, args=(r,)) for r in range(2)]
    [t.start() for t in ts]; [t.join() for t in ts]
    one = DistributedCheckpointManager(ProcessGroup.new_single_process(), str(tmp_path))
    with pytest.raises(RankMismatch):
        one.load(0)
    _, tensors, opt = one.load(0, allow_reshard=True)
    assert torch.equal(tensors["flat"], full) and opt is None
    assert torch.equal(reshard_flat([full[:5], full[5:]], 3, 2), torch.tensor([8.0, 9.0, 0.0, 0.0]))   # padded tail


def test_async_checkpoint_only_counts_after_finish(tmp_path):
    pg = ProcessGroup.new_single_process()
    mgr = DistributedCheckpointManager(pg, str(tmp_path))
    w = Parameter("w", _vec(1 << 16, 8))
    writer = AsyncCheckpointWriter()
    try:
        mgr.save_async(1, 42, [("w", w)], writer, {"t": 3})
        snapshot = w.tensor.clone()
        w.tensor.data.zero_()                                # training moves on while the file is written
        assert mgr.latest_checkpoint() is None               # no metadata yet
        mgr.finish_async(1, 42, writer)
        assert writer.pending() == 0 and writer.bytes_written() > 4 * (1 << 16)
    finally:
        writer.close()
    step, tensors, opt = mgr.load(1)
    assert step == 42 and opt == {"t": 3} and torch.equal(tensors["w"], snapshot)


def test_sharded_checkpoint_scatter_then_gather_is_identity():
    pgs = ProcessGroup.new_threaded(2)
    import threading
    full = _vec(12, 9).view(6, 2)
    out = [None, None]

    def run(rank):
        sc = ShardedCheckpoint(pgs[rank])
        out[rank] = sc.gather(sc.scatter(full))
    ts = [threading.Thread(target=run, args=(r,)) for r in range(2)]
    [t.start() for t in ts]; [t.join() for t in ts]
    assert torch.equal(out[0], full) and torch.equal(out[1], full)
