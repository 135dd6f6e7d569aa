"""Optimizers, learning-rate schedules and loss scaling, one test per component with closed-form expectations
(the unit tests of crates/optim/src/{lib,lr_scheduler,mixed_precision}.rs)."""
import math

import pytest
import torch

from rustral_b200.core import Parameter
from rustral_b200.optim import (Adam, AdamW, ConstantLR, CosineAnnealingLR, ExponentialLR, LinearWarmup, LossScaleScheduler,
                                MixedPrecisionOptimizer, OneCycleLR, PlateauLR, PolynomialLR, Sgd, StepDecay, WarmupCosine)


def _param(values):
    return Parameter("p", torch.tensor(values, dtype=torch.float32))


def test_sgd_plain_update_is_p_minus_lr_times_g():
    p = _param([1.0, -2.0, 0.5])
    g = torch.tensor([0.5, 0.25, -1.0])
    Sgd(0.1).step([p], {p.id: g})
    assert torch.allclose(p.tensor, torch.tensor([0.95, -2.025, 0.6]))


def test_sgd_momentum_accumulates_velocity():
    p = _param([0.0])
    opt = Sgd(1.0, momentum=0.5)
    g = torch.tensor([1.0])
    seen = []
    for _ in range(4):
        opt.step([p], {p.id: g})
        seen.append(float(p.tensor))
    # velocity 1, 1.5, 1.75, 1.875 -> positions -1, -2.5, -4.25, -6.125
    assert seen == pytest.approx([-1.0, -2.5, -4.25, -6.125])


def test_sgd_weight_decay_adds_lambda_p_to_the_gradient():
    p = _param([2.0])
    Sgd(0.1, weight_decay=0.5).step([p], {p.id: torch.tensor([0.0])})
    assert float(p.tensor) == pytest.approx(2.0 - 0.1 * 0.5 * 2.0)


def test_adam_first_step_moves_by_lr_in_the_gradient_direction():
    """With bias correction the first update is lr * g / (|g| + eps) whatever the gradient's size."""
    p = _param([0.0, 0.0, 0.0])
    g = torch.tensor([1e-3, -5.0, 200.0])
    Adam(0.01).step([p], {p.id: g})
    assert torch.allclose(p.tensor, torch.tensor([-0.01, 0.01, -0.01]), atol=1e-6)


def test_adam_matches_the_textbook_recurrence_over_several_steps():
    lr, b1, b2, eps = 0.05, 0.9, 0.999, 1e-8
    p = _param([1.0])
    opt = Adam(lr, b1, b2, eps)
    m = v = 0.0
    x = 1.0
    for t, g in enumerate([0.3, -0.2, 0.7, 0.1], start=1):
        opt.step([p], {p.id: torch.tensor([g])})
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        x -= lr * (m / (1 - b1 ** t)) / (math.sqrt(v / (1 - b2 ** t)) + eps)
        assert float(p.tensor) == pytest.approx(x, abs=1e-6)


def test_adamw_decay_is_decoupled_from_the_gradient_statistics():
    """AdamW shrinks the weight by lr * wd * p on top of the Adam step; coupled Adam feeds wd * p into the moments."""
    g = torch.tensor([0.0])
    pw, pc = _param([4.0]), _param([4.0])
    AdamW(0.1, weight_decay=0.5).step([pw], {pw.id: g})
    Adam(0.1, weight_decay=0.5, decoupled=False).step([pc], {pc.id: g})
    assert float(pw.tensor) == pytest.approx(4.0 - 0.1 * 0.5 * 4.0)          # zero gradient: only the decay moves it
    assert float(pc.tensor) == pytest.approx(4.0 - 0.1, abs=1e-5)            # decay acts as a gradient: a full Adam step


def test_optimizer_state_is_per_parameter_and_checkpointable():
    from rustral_b200.optim import MissingState
    a, b = Parameter("a", torch.ones(3)), Parameter("b", torch.ones(2))
    opt = Adam(0.01)
    opt.step([a, b], {a.id: torch.ones(3), b.id: -torch.ones(2)})
    opt.step([a], {a.id: torch.ones(3)})                              # a has taken two steps, b one
    ck = opt.save_checkpoint([("a", a), ("b", b)])
    assert ck.state["a"]["t"] == 2 and ck.state["b"]["t"] == 1 and len(ck.state["a"]["m"]) == 3
    a2, b2 = Parameter("a", a.tensor.clone()), Parameter("b", b.tensor.clone())
    opt2 = Adam(0.5)
    opt2.load_checkpoint(ck, [("a", a2), ("b", b2)])
    assert opt2.lr == 0.01
    opt.step([a, b], {a.id: torch.ones(3), b.id: torch.ones(2)})
    opt2.step([a2, b2], {a2.id: torch.ones(3), b2.id: torch.ones(2)})
    assert torch.equal(a.tensor, a2.tensor) and torch.equal(b.tensor, b2.tensor)
    with pytest.raises(MissingState):
        Adam(0.01).load_checkpoint(ck, [("c", Parameter("c", torch.ones(3)))])


# ---- schedules ------------------------------------------------------------------------------------------------------
def test_constant_and_linear_warmup():
    assert ConstantLR(0.3).get_lr(0) == ConstantLR(0.3).get_lr(10 ** 6) == 0.3
    w = LinearWarmup(0.0, 1.0, 10)
    assert [w.get_lr(s) for s in (0, 5, 10, 50)] == pytest.approx([0.0, 0.5, 1.0, 1.0])


def test_cosine_annealing_hits_its_end_points_and_midpoint():
    c = CosineAnnealingLR(1.0, 0.1, 100)
    assert c.get_lr(0) == pytest.approx(1.0) and c.get_lr(50) == pytest.approx(0.55) and c.get_lr(100) == pytest.approx(0.1)
    assert c.get_lr(1000) == pytest.approx(0.1)
    assert all(c.get_lr(s) >= c.get_lr(s + 1) for s in range(100))


def test_warmup_cosine_is_continuous_at_the_joint():
    s = WarmupCosine(1e-3, 1e-5, 10, 110)
    assert s.get_lr(0) == 0.0 and s.get_lr(5) == pytest.approx(5e-4) and s.get_lr(10) == pytest.approx(1e-3)
    assert s.get_lr(60) == pytest.approx(1e-5 + 0.5 * (1e-3 - 1e-5)) and s.get_lr(110) == pytest.approx(1e-5)
    assert abs(s.get_lr(9) - s.get_lr(10)) < 1.1e-4
    assert WarmupCosine(1.0, 0.0, 4, 8).with_initial_lr(0.2).get_lr(0) == 0.2


def test_step_exponential_and_polynomial_decay():
    assert [StepDecay(1.0, 0.5, 10).get_lr(s) for s in (0, 9, 10, 25, 30)] == [1.0, 1.0, 0.5, 0.25, 0.125]
    e = ExponentialLR(2.0, 0.1)
    assert e.get_lr(0) == 2.0 and e.get_lr(10) == pytest.approx(2.0 * math.exp(-1.0))
    p = PolynomialLR(1.0, 0.0, 10, power=2.0)
    assert p.get_lr(5) == pytest.approx(0.25) and p.get_lr(10) == 0.0 and p.get_lr(99) == 0.0


def test_one_cycle_rises_linearly_then_falls_on_a_cosine():
    o = OneCycleLR(1.0, 100)
    assert o.get_lr(0) == pytest.approx(0.1) and o.get_lr(25) == pytest.approx(0.55) and o.get_lr(50) == pytest.approx(1.0)
    assert o.get_lr(75) == pytest.approx(0.55) and o.get_lr(100) == pytest.approx(0.1)


def test_plateau_waits_for_patience_respects_cooldown_and_floor():
    pl = PlateauLR(1.0, min_lr=0.2, factor=0.5, patience=2, cooldown=1)
    lrs = [pl.report_loss(l) for l in (1.0, 0.9, 0.9, 0.9, 0.9)]
    assert lrs == [1.0, 1.0, 1.0, 1.0, 0.5]                  # improvement, then three non-improving reports > patience 2
    assert pl.report_loss(0.9) == 0.5                         # cooldown swallows one report
    for _ in range(3):
        pl.report_loss(0.9)
    assert pl.current_lr() == 0.25
    for _ in range(10):
        pl.report_loss(0.9)
    assert pl.current_lr() == 0.2                             # never below min_lr
    pl.reset()
    assert pl.current_lr() == 1.0


def test_scheduler_drives_an_attached_optimizer():
    opt = Sgd(123.0)
    sched = StepDecay(1.0, 0.1, 2).attach(opt)
    assert opt.lr == 1.0
    seen = [sched.step() for _ in range(4)]
    assert seen == pytest.approx([1.0, 0.1, 0.1, 0.01]) and opt.lr == pytest.approx(0.01)
    sched.reset()
    assert sched.current_lr() == 1.0 and sched.name() == "StepDecay"


# ---- loss scaling ---------------------------------------------------------------------------------------------------
def test_loss_scale_halves_on_overflow_and_doubles_after_clean_interval():
    ls = LossScaleScheduler(1024.0, growth_interval=3)
    assert ls.step(True) and ls.scale == 512.0                # overflow: skip the step, halve
    assert [ls.step(False) for _ in range(3)] == [False, False, False] and ls.scale == 1024.0
    assert ls.step(True) and ls.step(True) and ls.scale == 256.0


def test_mixed_precision_optimizer_unscales_and_skips_overflowed_steps():
    g = torch.tensor([0.5, -0.25])
    p, q = _param([1.0, 1.0]), _param([1.0, 1.0])
    mp = MixedPrecisionOptimizer(Sgd(0.1), loss_scale=LossScaleScheduler(16.0))
    assert mp.step([p], {p.id: g * 16.0})
    Sgd(0.1).step([q], {q.id: g})
    assert torch.allclose(p.tensor, q.tensor)
    before = p.tensor.clone()
    assert not mp.step([p], {p.id: torch.tensor([float("nan"), 1.0])})
    assert torch.equal(p.tensor, before) and mp.skipped_steps == 1 and mp.loss_scale.scale == 8.0
    assert float(mp.scale_loss(torch.tensor(2.0))) == 16.0
