"""Regression cases for faults found by review: each test fails on the code before its fix."""
import threading

import pytest
import torch

from rustral_b200.core.parameter import Parameter
from rustral_b200.models.config import preset
from rustral_b200.optim import Adam, AdamCheckpoint
from rustral_b200.serve.engine import ServingEngine
from rustral_b200.serve.model_runner import ModelRunner
from rustral_b200.serve.scheduler import PyScheduler, Scheduler


# ---------------------------------------------------------------------------------------------- optimizer master copies
def _lowp_param(seed=0, n=64):
    g = torch.Generator().manual_seed(seed)
    return Parameter("w", torch.randn(n, generator=g).to(torch.bfloat16))


def test_adam_uses_weights_loaded_after_its_first_step():
    """A state-dict load (an in-place write by somebody else) after the first step must not be reverted by the
    optimizer's fp32 master copy at the next step."""
    p = _lowp_param()
    opt = Adam(lr=1e-2)
    g = torch.ones(64)
    opt.step([p], {p.id: g})
    loaded = torch.full((64,), 3.0, dtype=torch.bfloat16)
    with torch.no_grad():
        p.tensor.copy_(loaded)                               # e.g. load_state_dict
    opt.step([p], {p.id: g})
    # the step moved the LOADED weights by about lr, it did not jump back to the pre-load trajectory
    assert (p.tensor.float() - 3.0).abs().max() < 0.05
    # and an explicit reset does the same for writes the version counter cannot see
    p.tensor.data = torch.full((64,), -2.0, dtype=torch.bfloat16)
    opt.reset_master([p])
    opt.step([p], {p.id: g})
    assert (p.tensor.float() + 2.0).abs().max() < 0.05


def test_adam_master_is_not_rederived_without_external_writes():
    """Without outside writes the fp32 master keeps the bits bf16 cannot hold: many tiny steps accumulate."""
    p = Parameter("w", torch.ones(8, dtype=torch.bfloat16))
    opt = Adam(lr=1e-4)                                       # 1e-4 is below bf16 resolution at 1.0 (2^-8)
    for _ in range(60):
        opt.step([p], {p.id: torch.ones(8)})
    master = opt._master[p.id]
    assert float(master[0]) < 1.0 - 50e-4                     # the fp32 copy moved ...
    assert float(p.tensor[0]) < 1.0                           # ... and eventually so did the rounded copy


def test_adam_checkpoint_carries_the_master_copy():
    """A resumed run continues the uninterrupted run bit for bit: the fp32 master copy is part of the checkpoint."""
    g = torch.Generator().manual_seed(3)
    grads = [torch.randn(64, generator=g) for _ in range(6)]
    a = _lowp_param(1)
    opt_a = Adam.adamw(lr=3e-3, weight_decay=0.1)
    for gr in grads[:3]:
        opt_a.step([a], {a.id: gr})
    ck = AdamCheckpoint.from_json(opt_a.save_checkpoint([("w", a)]).to_json())
    assert "master" in ck.state["w"]
    b = Parameter("w", a.tensor.clone())
    opt_b = Adam.adamw(lr=1.0)
    opt_b.load_checkpoint(ck, [("w", b)])
    for gr in grads[3:]:
        opt_a.step([a], {a.id: gr})
        opt_b.step([b], {b.id: gr})
    assert torch.equal(a.tensor, b.tensor)
    assert torch.equal(opt_a._master[a.id], opt_b._master[b.id])


# ---------------------------------------------------------------------------------------------- serving admission
def _engine(num_blocks=4, seq_len=256):
    cfg = preset("gpt2-test", seq_len=seq_len, d_model=64, ffn_dim=128)
    return ServingEngine(ModelRunner(cfg, device="cpu", num_blocks=num_blocks), max_batch_size=4)


def test_submit_refuses_requests_that_can_never_fit_the_cache():
    eng = _engine(num_blocks=4)                               # 4 blocks of 16 tokens
    with pytest.raises(ValueError, match="KV blocks"):
        eng.submit(list(range(1, 60)), 20)                    # 59 + 20 + 1 tokens = 5 blocks
    with pytest.raises(ValueError, match="max_tokens"):
        eng.submit([1, 2, 3], 0)
    assert not eng.scheduler.has_work()
    # a request that does fit still runs, and nothing is left behind
    assert len(eng.generate([1, 2, 3], 4)) == 4
    assert eng.runner.cache.free_blocks == 4


@pytest.mark.parametrize("cls", [PyScheduler, Scheduler])
def test_scheduler_abort_frees_blocks_in_every_queue(cls):
    from rustral_b200.serve.kv_cache import PagedCache
    cache = PagedCache(8, 16)
    s = cls(cache, max_batch_size=2)
    ids = [s.add_request(list(range(20)), 4) for _ in range(4)]
    batch = s.schedule()                                      # two admitted (2 blocks each), two pending
    assert len(batch) == 2 and cache.free_blocks == 4
    assert s.abort(ids[0]) and s.abort(ids[3])
    assert cache.free_blocks == 6
    assert not s.abort(12345)
    s.abort(ids[1]); s.abort(ids[2])
    assert not s.has_work() and cache.free_blocks == 8


def test_engine_loop_drops_the_requests_of_a_failed_step():
    """When the model step raises, the waiting handlers get the error, the requests leave the scheduler (the loop does
    not retry the failing step for ever) and the loop keeps serving."""
    from rustral_b200.serve.http_server import EngineLoop
    eng = _engine(num_blocks=32, seq_len=64)
    real_pass = eng.runner.step_mixed
    calls = {"n": 0}

    def flaky(*args):
        calls["n"] += 1
        if calls["n"] == 1:
            raise RuntimeError("injected model failure")
        return real_pass(*args)
    eng.runner.step_mixed = flaky
    loop = EngineLoop(eng)
    try:
        with pytest.raises(RuntimeError, match="injected"):
            loop.generate([1, 2, 3], 4, timeout=60)
        assert loop.failed_steps == 1
        deadline = threading.Event()
        deadline.wait(0.2)
        assert not eng.scheduler.has_work() and eng.runner.cache.free_blocks == 32
        assert len(loop.generate([1, 2, 3], 4, timeout=60)) == 4       # still alive, step no longer failing
        assert calls["n"] == 2
    finally:
        loop.shutdown()


def test_trainer_updates_parameters_that_the_model_put_on_the_tape_itself():
    """A model whose forward_tape brings its parameters onto the tape with watch_parameter() trains through the Trainer
    builder: the gradients land on the tape's leaves, not on `parameter.tensor.grad`, and the trainer must collect them
    from there (it used to step with no gradients at all, leaving such a model at its initial loss)."""
    import torch
    from rustral_b200.core import CpuBackend
    from rustral_b200.core.module import Module, Trainable
    from rustral_b200.nn import LinearBuilder
    from rustral_b200.optim import Sgd
    from rustral_b200.runtime.tape_trainer import SupervisedTapeModel, Trainer
    be = CpuBackend()

    class M(Module, Trainable, SupervisedTapeModel):
        def __init__(self):
            self.lin = LinearBuilder(2, 2).with_bias().seed(1).build(be)

        def forward_tape(self, x, tape, ctx):
            return tape.linear_tape(tape.constant(x), tape.watch_parameter(self.lin.weight), tape.watch_parameter(self.lin.bias))
    m = M()
    before = m.lin.weight.tensor.detach().clone()
    data = [([1.0, 0.0], 0), ([0.0, 1.0], 1)] * 4
    rep = Trainer.classification(Sgd(0.5)).epochs(20).batch_size(4).fit(be, m, data)
    assert not torch.equal(before, m.lin.weight.tensor.detach())
    assert rep.epochs[-1].mean_loss < 0.5 * rep.epochs[0].mean_loss and rep.accuracy == 1.0


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("act", ["none", "gelu", "dgelu"])
def test_padded_gemm_path_gives_the_same_result_as_the_direct_one(a_mn, b_mn, act):
    """Layer sizes the kernel cannot address (2 -> 8, 10 classes, 3x3 filters over one channel) run on zero-padded copies;
    the padding and the copy back are checked here against the direct product, for every operand layout, with bias,
    residual, saved pre-activation, activation-gradient input, scales and accumulation."""
    import torch
    from rustral_b200.ops import matmul as mm
    g = torch.Generator().manual_seed(3)
    M, N, K = 5, 10, 3
    a = torch.randn((K, M) if a_mn else (M, K), generator=g)
    b = torch.randn((K, N) if b_mn else (N, K), generator=g)
    bias, res, aux = torch.randn(N, generator=g), torch.randn(M, N, generator=g), torch.randn(M, N, generator=g)
    rs, cs = torch.rand(M, generator=g) + 0.5, torch.rand(N, generator=g) + 0.5
    kw = dict(a_mn=a_mn, b_mn=b_mn, bias=bias, act=act, residual=res, aux_in=aux if act == "dgelu" else None, alpha=0.7)
    seen = {}

    def spy(ap, bp, **k):
        seen["shapes"] = (tuple(ap.shape), tuple(bp.shape), tuple(k["out"].shape), k["bias"].shape[0])
        return mm.gemm(ap, bp, **k)
    for accumulate in (False, True):
        want_aux = torch.zeros(M, N) if act == "gelu" else None
        got_aux = torch.zeros(M, N) if act == "gelu" else None
        out0 = torch.randn(M, N, generator=torch.Generator().manual_seed(9))
        want = mm.gemm(a, b, **kw, aux_out=want_aux, out=out0.clone(), accumulate=accumulate, row_scale=rs, col_scale=cs)
        got = mm._gemm_padded(a, b, **kw, aux_out=got_aux, out=out0.clone(), out_dtype=torch.float32, accumulate=accumulate,
                              row_scale=rs, col_scale=cs, call=spy)
        assert torch.allclose(got, want, atol=1e-5)
        if act == "gelu":
            assert torch.allclose(got_aux, want_aux, atol=1e-5)
    M8 = 8 if a_mn else 5
    assert seen["shapes"] == ((8, M8) if a_mn else (5, 8), (8, 16) if b_mn else (16, 8), (M8, 16), 16)
    fresh = mm._gemm_padded(a, b, **kw, aux_out=None, out=None, out_dtype=torch.float32, accumulate=False, row_scale=None,
                            col_scale=None)
    assert fresh.shape == (M, N) and fresh.is_contiguous()
    assert torch.allclose(fresh, mm.gemm(a, b, **kw), atol=1e-5)


def test_alignment_check_flags_exactly_the_shapes_the_kernel_cannot_address():
    import torch
    from rustral_b200.ops.matmul import _needs_padding
    bf = torch.bfloat16
    ok_a, ok_b = torch.zeros(32, 64, dtype=bf), torch.zeros(48, 64, dtype=bf)
    assert not _needs_padding(ok_a, ok_b, None, None, None, None, None, bf, 48)
    assert _needs_padding(torch.zeros(4, 2, dtype=bf), torch.zeros(8, 2, dtype=bf), None, None, None, None, None, bf, 8)     # K = 2
    assert _needs_padding(ok_a, torch.zeros(10, 64, dtype=bf), None, None, None, None, None, bf, 10)                        # N = 10
    assert not _needs_padding(ok_a, torch.zeros(12, 64, dtype=bf), None, None, None, None, None, torch.float32, 12)          # fp32 rows of 12 are fine
    assert _needs_padding(ok_a, ok_b, None, torch.zeros(32, 50, dtype=bf)[:, :48], None, None, None, bf, 48)                # residual pitch 50
    assert _needs_padding(ok_a[:, 1:], ok_b[:, 1:], None, None, None, None, None, bf, 48)                                   # bases off by 2 bytes
    assert _needs_padding(ok_a, ok_b, torch.zeros(49, dtype=bf)[1:], None, None, None, None, bf, 48)                        # bias base
    assert _needs_padding(ok_a, ok_b, None, None, None, None, torch.zeros(32, 52, dtype=bf)[:, :48], bf, 48)               # given output
