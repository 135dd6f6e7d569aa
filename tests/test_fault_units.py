"""Failure detection, elastic recovery and seeded fault injection, component by component, all on the host
(crates/distributed/src/fault_tolerance.rs and chaos_engineering.rs `mod tests`).  No GPU, no device fault: a failure is a
rank that stops reporting, an exception from a step, or a flag from the seeded scheduler."""
import pytest

from rustral_b200.parallel.chaos_engineering import (ChaosMonkey, ChaosScenarios, CheckpointCorruption, FaultInjection, FaultKind,
                                                     FaultType, corrupt_checkpoint_file)
from rustral_b200.parallel.fault_tolerance import (CheckpointVersion, DictStore, ElasticProcessGroup, ElasticTrainer, HealthMonitor,
                                                   MemoryCheckpointStore, NodeState, RestartConfig, StateSync, TimedBarrier)
from rustral_b200.parallel.process_group import CommunicationError, DistributedError, ProcessGroup


class _Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        return self.t


def test_health_monitor_state_machine_and_recovery_from_suspicion():
    clk = _Clock()
    h = HealthMonitor(0, timeout_ms=1000.0, clock=clk)
    for r in range(3):
        h.register_node(r)
    clk.t = 1.5
    h.heartbeat(0); h.heartbeat(1)
    assert h.check_health() == [] and h.nodes[2].state is NodeState.SUSPECTED and h.healthy_nodes() == [0, 1]
    h.heartbeat(2)                                             # it was only slow
    assert h.nodes[2].state is NodeState.HEALTHY
    clk.t = 4.0
    h.heartbeat(0)
    assert sorted(h.check_health()) == [1, 2] and h.check_health() == []      # reported once
    h.heartbeat(1)
    assert h.nodes[1].state is NodeState.FAILED                # a failed node does not come back by itself
    h.checkpoint_completed(0, 7)
    assert h.nodes[0].last_checkpoint == 7


def test_heartbeats_travel_through_the_store_between_monitors():
    clk, store = _Clock(), DictStore()
    a, b = (HealthMonitor(r, 1000.0, store, clk) for r in (0, 1))
    for m in (a, b):
        m.register_node(0); m.register_node(1)
    clk.t = 0.9
    b.heartbeat()
    clk.t = 1.5
    a.heartbeat()
    assert a.check_health() == [] and a.nodes[1].state is NodeState.HEALTHY    # b's beat at 0.9 was read from the store
    clk.t = 3.5
    a.heartbeat()
    assert a.check_health() == [1]


def test_elastic_group_shrinks_and_renumbers_the_survivors():
    clk = _Clock()
    pgs = ProcessGroup.new_threaded(4)
    h = HealthMonitor(2, 1000.0, clock=clk)
    g = ElasticProcessGroup(pgs[2], h)
    assert g.effective_world_size() == 4 and g.check_membership() is None
    clk.t = 5.0
    for r in (0, 2, 3):
        h.heartbeat(r)
    change = g.check_membership()
    assert change.kind == "nodes_failed" and change.ranks == [1] and not g.is_active(1) and g.effective_world_size() == 3
    rc = g.reconfigure()
    assert rc.kind == "reconfiguration_complete" and rc.ranks == [0, 2, 3] and rc.new_world_size == 3 and rc.new_rank == 1


def test_elastic_trainer_rolls_back_to_the_last_checkpoint_and_counts_lost_steps():
    store = MemoryCheckpointStore()
    tr = ElasticTrainer(store, max_retries=2, checkpoint_every=2)
    fail_at = {3}

    def step(i, state):
        if i in fail_at:
            fail_at.discard(i)
            raise CommunicationError("peer lost")
        return state + [i]
    out = tr.train_loop(step, 6, [])
    assert out == [0, 1, 2, 3, 4, 5]                            # step 2 was replayed after the rollback to the checkpoint at 2
    assert (tr.stats.failures, tr.stats.recoveries, tr.stats.lost_steps) == (1, 1, 1) and store.latest() == 6


def test_elastic_trainer_gives_up_after_max_retries_and_honours_the_restart_delay():
    slept = []
    tr = ElasticTrainer(MemoryCheckpointStore(), max_retries=2, sleep=slept.append, restart=RestartConfig(restart_delay_s=0.25))

    def always(i, s):
        raise CommunicationError("down")
    with pytest.raises(DistributedError):
        tr.train_loop(always, 3, 0)
    assert tr.stats.failures == 3 and slept == [0.25, 0.25]


def test_timed_barrier_and_state_sync():
    clk = _Clock()
    bar = TimedBarrier(3, 2.0, clk)
    bar.arrive(0); bar.arrive(2)
    assert not bar.is_complete() and bar.missing() == [1] and not bar.timed_out()
    clk.t = 2.5
    assert bar.timed_out()
    bar.arrive(1)
    assert bar.is_complete() and not bar.timed_out()
    bar.reset()
    assert bar.missing() == [0, 1, 2]
    sync = StateSync(3, min_nodes=2)
    sync.report(0, CheckpointVersion(1, 10))
    assert not sync.can_proceed()
    sync.report(1, CheckpointVersion(1, 10))
    assert sync.can_proceed() and not sync.is_complete()
    sync.report(2, CheckpointVersion(1, 8))
    assert not sync.can_proceed()                                # one node loaded another version
    sync.report(2, CheckpointVersion(1, 10))
    assert sync.is_complete()


# ---- seeded fault scheduler -----------------------------------------------------------------------------------------
def test_fault_injection_respects_delay_probability_and_trigger_cap():
    import random
    inj = FaultInjection(FaultType(FaultKind.SLOW_WORKER, delay_ms=5.0), 1.0, trigger_delay_ticks=3, max_triggers=2)
    rng = random.Random(0)
    assert not inj.should_trigger(rng, 2) and inj.should_trigger(rng, 3)
    inj.triggers = 2
    assert not inj.should_trigger(rng, 10)
    assert not FaultInjection(FaultType(FaultKind.PACKET_LOSS), 0.0).should_trigger(rng, 100)


def test_chaos_monkey_is_deterministic_for_a_seed_and_recovers_expired_faults():
    def run(seed):
        m = ChaosScenarios.random_stress(4, seed)
        log = []
        for _ in range(200):
            log.append([(r.fault.kind, r.ranks) for r in m.tick()])
        return m, log
    (m1, a), (_, b), (_, c) = run(5), run(5), run(6)
    assert a == b and a != c
    rep = m1.generate_report()
    assert rep.ticks == 200 and rep.faults_triggered == sum(len(x) for x in a) > 0
    assert 0 < rep.faults_recovered <= rep.faults_triggered and sum(rep.by_kind.values()) == rep.faults_triggered


def test_partition_blocks_only_traffic_across_the_cut():
    m = ChaosMonkey(1, 4)
    m.add_injection(FaultInjection(FaultType(FaultKind.NETWORK_PARTITION, ranks=(0, 1)), 1.0, duration_ticks=2, max_triggers=1))
    assert m.can_communicate(0, 3)
    m.tick()
    assert not m.can_communicate(0, 3) and m.can_communicate(0, 1) and m.can_communicate(2, 3) and m.is_rank_affected(1)
    m.tick(); m.tick()
    assert m.can_communicate(0, 3) and not m.is_rank_affected(1)


def test_slow_worker_and_crash_scenarios_act_through_run_with_faults():
    slept = []
    m = ChaosScenarios.slow_worker(2, rank=1, delay_ms=40.0)
    assert m.run_with_faults(lambda: "ok", rank=1, sleep=slept.append) == "ok" and slept == [0.04]
    assert m.run_with_faults(lambda: "ok", rank=0, sleep=slept.append) == "ok" and slept == [0.04] and m.get_delay_ms(1) == 40.0
    c = ChaosScenarios.cascading_failure(4)
    outcomes = []
    for _ in range(8):
        try:
            c.run_with_faults(lambda: None, rank=0)
            outcomes.append("ok")
        except CommunicationError:
            outcomes.append("down")
    assert outcomes[0] == "ok" and "down" in outcomes and outcomes[-1] == "ok"   # rank 0 crashes at tick 2 for three ticks


def test_packet_loss_rate_is_close_to_the_configured_rate():
    m = ChaosMonkey(3, 2)
    m.add_injection(FaultInjection(FaultType(FaultKind.PACKET_LOSS, loss_rate=0.25, ranks=(0,)), 1.0, duration_ticks=10 ** 6, max_triggers=1))
    m.tick()
    lost = sum(m.packet_lost(0, 1) for _ in range(4000))
    assert 800 < lost < 1200 and not any(ChaosMonkey(3, 2).packet_lost(0, 1) for _ in range(10))


@pytest.mark.parametrize("how", list(CheckpointCorruption))
def test_corrupted_checkpoints_are_rejected_by_the_loader(tmp_path, how):
    import torch
    from rustral_b200.core import CpuBackend
    from rustral_b200.core.errors import SerializationError
    from rustral_b200.nn import LinearBuilder
    from rustral_b200.runtime.model_io import load_model, save_model
    lin = LinearBuilder(8, 4).with_bias().seed(1).build(CpuBackend())
    path = tmp_path / "m.safetensors"
    path.write_bytes(save_model(lin))
    corrupt_checkpoint_file(str(path), how, seed=2)
    other = LinearBuilder(8, 4).with_bias().seed(9).build(CpuBackend())
    before = [p.tensor.clone() for p in other.parameters()]
    try:
        load_model(other, path.read_bytes())
        loaded = True
    except (SerializationError, Exception):      # noqa: BLE001 - any refusal counts; silent acceptance is checked below
        loaded = False
    if how in (CheckpointCorruption.TRUNCATED, CheckpointCorruption.MISSING_KEYS):
        assert not loaded and all(torch.equal(a, p.tensor) for a, p in zip(before, other.parameters()))   # nothing was written
