"""Core contracts one by one (crates/core/src/{parameter,module,shape,context,numerics,tolerance}.rs `mod tests`)."""
import threading

import pytest
import torch

from rustral_b200.core import (CpuBackend, DType, ForwardCtx, InvalidShape, Mode, Module, NumericsConfig, NumericsValidator,
                               OpFamily, OperationProfiler, Parameter, ParameterGroup, ParameterId, ParameterRef, Saveable,
                               SerializationError, Shape, ShapeMismatch, ShapePolicy, Tolerance, ToleranceConfig, Trainable,
                               assert_close, assert_slices_close, collect_named_parameter_ids, collect_named_parameters)
from rustral_b200.nn import ExpertChoiceConfig, LinearBuilder, RoutingComparison

BE = CpuBackend()


# ---- parameters -----------------------------------------------------------------------------------------------------
def test_parameter_ids_are_unique_across_threads_and_survive_a_storage_swap():
    ids = []

    def make():
        ids.extend(int(Parameter("p", torch.zeros(1)).id) for _ in range(200))
    ts = [threading.Thread(target=make) for _ in range(4)]
    [t.start() for t in ts]; [t.join() for t in ts]
    assert len(set(ids)) == 800
    p = Parameter("w", torch.ones(2, 3))
    q = Parameter.with_tensor(p, torch.zeros(2, 3))
    assert q.id == p.id and q.name == "w" and q.tensor.requires_grad and float(q.tensor.sum()) == 0.0
    assert isinstance(ParameterId.fresh(), int) and ParameterRef(p).id == p.id and ParameterRef(p).name == "w"
    assert "shape=(2, 3)" in repr(p)


def test_parameter_set_checks_the_shape_and_integer_tensors_take_no_gradient():
    p = Parameter("w", torch.zeros(2, 2))
    p.set_(torch.ones(2, 2, dtype=torch.float64))
    assert p.tensor.dtype == torch.float32 and float(p.tensor.sum()) == 4.0 and p.tensor.requires_grad
    with pytest.raises(ShapeMismatch):
        p.set_(torch.ones(3, 2))
    assert not Parameter("ids", torch.zeros(3, dtype=torch.int64)).tensor.requires_grad
    assert not Parameter("frozen", torch.zeros(3), requires_grad=False).tensor.requires_grad
    (p.tensor * 2).sum().backward()
    assert torch.equal(p.grad, torch.full((2, 2), 2.0))
    p.zero_grad()
    assert p.grad is None
    p.to(torch.float64)
    assert p.tensor.dtype == torch.float64 and p.tensor.requires_grad and p.tensor.is_leaf


def test_parameter_groups_carry_hyper_parameters():
    a, b = Parameter("a", torch.zeros(3)), Parameter("b", torch.zeros(2, 2))
    g = ParameterGroup("no_decay", [a], weight_decay=0.0, lr=1e-3)
    g.add(b)
    assert len(g) == 2 and g.numel() == 7 and [p.name for p in g] == ["a", "b"] and g.hyper == {"weight_decay": 0.0, "lr": 1e-3}


# ---- module traits --------------------------------------------------------------------------------------------------
class _Leaf(Module, Trainable, Saveable):
    def __init__(self, seed):
        self.weight = BE.normal_parameter("weight", (2, 2), seed, 1.0)
        self._hidden = BE.normal_parameter("hidden", (2,), seed, 1.0)       # underscore: not enumerated
        self.note = "not a parameter"

    def forward(self, x, ctx):
        return x @ self.weight.tensor


class _Tree(Module, Trainable, Saveable):
    def __init__(self):
        self.first = _Leaf(1)
        self.stack = [_Leaf(2), _Leaf(3)]
        self.scales = [BE.constant_parameter("s", (1,), 1.0), BE.constant_parameter("s", (1,), 2.0)]
        self.empty = []

    def forward(self, x, ctx):
        for m in [self.first] + self.stack:
            x = m(x, ctx)
        return x * self.scales[0].tensor * self.scales[1].tensor


def test_named_parameters_follow_attribute_order_with_list_indices():
    t = _Tree()
    names = [n for n, _ in t.named_parameters()]
    assert names == ["first.weight", "stack.0.weight", "stack.1.weight", "scales.0", "scales.1"]
    assert collect_named_parameters(t)[0][0] == "first.weight" and set(collect_named_parameter_ids(t)) == set(names)
    assert t.num_parameters() == 14 and len(t.parameters()) == 5
    seen = []
    t.visit_parameters(lambda n, p: seen.append(n), prefix="model.")
    assert seen[0] == "model.first.weight" and seen[-1] == "model.scales.1"
    y = t(torch.ones(1, 2))                                   # __call__ without a context means inference
    y.sum().backward()
    assert all(p.grad is not None for p in t.parameters())
    t.zero_grad()
    assert all(p.grad is None for p in t.parameters())


def test_state_dict_round_trip_is_strict_and_atomic():
    a, b = _Tree(), _Tree()
    with torch.no_grad():
        for p in a.parameters():
            p.tensor.add_(1.0)
    sd = a.state_dict()
    sd["first.weight"].zero_()                                # the state dict holds copies
    assert float(a.first.weight.tensor.abs().sum()) > 0
    sd = a.state_dict()
    b.load_state_dict(sd)
    assert all(torch.equal(x.tensor, y.tensor) for x, y in zip(a.parameters(), b.parameters()))
    before = [p.tensor.clone() for p in b.parameters()]
    bad = dict(sd)
    bad["stack.1.weight"] = torch.zeros(3, 3)
    bad["first.weight"] = torch.full((2, 2), 9.0)
    with pytest.raises(ShapeMismatch):
        b.load_state_dict(bad)
    assert all(torch.equal(x, p.tensor) for x, p in zip(before, b.parameters()))      # nothing was half-loaded
    with pytest.raises(SerializationError, match="missing"):
        b.load_state_dict({k: v for k, v in sd.items() if k != "scales.1"})
    with pytest.raises(SerializationError, match="unexpected"):
        b.load_state_dict({**sd, "extra": torch.zeros(1)})
    b.load_state_dict({"first.weight": torch.zeros(2, 2)}, strict=False)
    assert float(b.first.weight.tensor.abs().sum()) == 0.0


# ---- shapes, context ------------------------------------------------------------------------------------------------
def test_shape_validation_and_policy():
    s = Shape([2, 3, 4])
    assert s.rank == 3 and s.numel() == 24 and list(s) == [2, 3, 4] and s[1] == 3 and len(s) == 3 and s == Shape((2, 3, 4))
    for bad in ([], [2, 0], [-1]):
        with pytest.raises(InvalidShape):
            Shape(bad)
    assert ShapePolicy.STATIC.supports_cuda_graph_capture() and not ShapePolicy.DYNAMIC_BOUNDED.supports_cuda_graph_capture()
    assert ShapePolicy.DYNAMIC_BOUNDED.prefers_arena_pool() and not ShapePolicy.DYNAMIC_UNBOUNDED.prefers_arena_pool()


def test_forward_ctx_modes_run_ids_profiler_and_rng_ranges():
    a, b = ForwardCtx.train(BE, seed=5), ForwardCtx.inference(BE)
    assert a.is_training() and a.mode is Mode.TRAIN and not b.is_training() and b.run_id > a.run_id and a.seed == 5
    assert a.next_rng_offset(10) == 0 and a.next_rng_offset(4) == 10 and a.next_rng_offset(1) == 14
    with b.profile("noop", (1,)):                              # no profiler attached: a no-op guard
        pass
    prof = OperationProfiler(use_cuda_events=False)
    c = ForwardCtx.inference(BE).with_profiler(prof).with_shape_policy(ShapePolicy.STATIC)
    lin = LinearBuilder(4, 4).build(BE)
    with c.profile("my_block", (2, 4)):
        lin(torch.zeros(2, 4), c)
    assert c.shape_policy is ShapePolicy.STATIC and prof.stats["my_block"].count == 1
    assert prof.stats["linear"].count == 1 and prof.stats["my_block"].total_ms >= prof.stats["linear"].total_ms   # the layer records itself


# ---- numerics -------------------------------------------------------------------------------------------------------
def test_tolerances_validator_and_assertions():
    assert Tolerance(1e-3, 1e-6).is_close(1.0005, 1.0) and not Tolerance(1e-3, 1e-6).is_close(1.002, 1.0)
    cfg = NumericsConfig()
    assert cfg.for_dtype(DType.F32) == Tolerance(1e-5, 1e-8) and cfg.for_dtype(DType.BF16).max_ulps == 4
    ref = torch.linspace(1, 2, 200)
    off = ref.clone()
    off[0] += 1e-2
    lax, strict = NumericsValidator(), NumericsValidator(NumericsConfig(strict=True))
    r = lax.validate_arrays(off, ref)
    assert r.ok and r.violations == 1 and r.total == 200 and r.max_abs_err == pytest.approx(1e-2, rel=1e-3)   # 1 of 200 is within 1 %
    assert not strict.validate_arrays(off, ref).ok
    off[1:4] += 1e-2
    assert not lax.validate_arrays(off, ref).ok                                                    # 4 of 200 is not
    assert lax.validate_arrays(off, ref, DType.BF16).ok                                            # but fine at bf16 tolerance
    nan = ref.clone(); nan[5] = float("nan")
    rep = lax.validate_arrays(nan, ref)
    assert rep.has_nan and not rep.ok
    assert not lax.validate_arrays(ref[:10], ref).ok                                               # length mismatch
    assert ToleranceConfig.for_family(OpFamily.MATMUL) == Tolerance(1e-4, 1e-5)
    assert ToleranceConfig.for_family(OpFamily.ATTENTION, DType.BF16).rtol == 3e-2
    assert_close([1.0, 2.0], [1.0, 2.0 + 1e-9])
    assert assert_slices_close is assert_close
    with pytest.raises(AssertionError, match="1 of 2 elements differ; first at flat index 1"):
        assert_close([1.0, 2.0], [1.0, 2.1], what="row")
    with pytest.raises(AssertionError, match="shape"):
        assert_close([1.0], [1.0, 2.0])


def test_routing_comparison_is_the_load_formula():
    c = RoutingComparison.compare(num_tokens=1000, num_experts=8, top_k=2, observed_max_fraction=0.3)
    assert c.token_choice_max_load == pytest.approx(600.0) and c.expert_choice_max_load == pytest.approx(250.0)
    assert ExpertChoiceConfig(16, 4, 32, tokens_per_expert=8).tokens_per_expert == 8


def test_parallel_reductions_switch(monkeypatch):
    from rustral_b200 import ops
    from rustral_b200.core import PAR_REDUCE_ENV, PARALLEL_REDUCTIONS_ENV, parallel_reductions_enabled
    monkeypatch.delenv(PARALLEL_REDUCTIONS_ENV, raising=False)
    monkeypatch.delenv(PAR_REDUCE_ENV, raising=False)
    assert not parallel_reductions_enabled()
    x = torch.full((1 << 20,), 0.1) * torch.arange(1, (1 << 20) + 1).float().reciprocal()
    exact = float(x.double().sum())
    serial = float(ops.sum_all(x))
    assert serial == float(torch.tensor(exact, dtype=torch.float64).float())        # the float64 sum rounded once
    assert float(ops.sum_dim0(x.view(1 << 10, 1 << 10)).sum()) == pytest.approx(exact, rel=1e-6)
    monkeypatch.setenv(PAR_REDUCE_ENV, "1")
    assert parallel_reductions_enabled()
    assert float(ops.sum_all(x)) == pytest.approx(exact, rel=1e-5)                  # plain fp32 sum: close, not necessarily equal
    monkeypatch.setenv(PAR_REDUCE_ENV, "0")
    monkeypatch.setenv(PARALLEL_REDUCTIONS_ENV, "1")
    assert parallel_reductions_enabled()
