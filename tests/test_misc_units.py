"""Components that the other unit-test files do not reach: shared + routed experts, the token sampler, the model
registry, the JSON-lines event writer behind the trainer's metrics, and the tensor pool / memory profiler pair
(crates/nn/src/shared_expert.rs, continuous_batching.rs:454-490, crates/model-zoo, crates/metrics, crates/core `mod tests`)."""
import json

import pytest
import torch

from rustral_b200.core import CpuBackend, ForwardCtx, MemoryProfiler, PoolStrategy, TensorPool
from rustral_b200.nn import SharedAndRoutedConfig, SharedExpertConfig, SharedExpertLayer
from rustral_b200.serve.sampler import Sampler

BE = CpuBackend()


# ---- shared + routed experts ----------------------------------------------------------------------------------------
def test_shared_expert_layer_is_residual_plus_shared_plus_weighted_routed_part():
    cfg = SharedExpertConfig(d_model=16, num_shared=2, num_routed=4, expert_hidden_dim=24, top_k=2)
    layer = SharedExpertLayer.new(BE, cfg, seed=3)
    x = torch.randn(5, 7, 16, generator=torch.Generator().manual_seed(0))
    ctx = ForwardCtx.inference(BE)
    y = layer(x, ctx)
    assert y.shape == x.shape
    # rebuild the output from the parts with plain tensor math
    x2 = x.reshape(-1, 16)
    shared = sum(e(x2, ctx) for e in layer.shared_experts) / 2
    probs = torch.softmax(x2 @ layer.router.tensor.t(), -1)
    w, idx = probs.topk(2, -1)
    routed = torch.zeros_like(x2)
    for t in range(x2.shape[0]):
        for k in range(2):
            e = int(idx[t, k])
            gu = layer.routed_w1.tensor[e] @ x2[t]
            g, u = gu[:24], gu[24:]
            routed[t] += w[t, k] * (layer.routed_w2.tensor[e] @ (torch.nn.functional.silu(g) * u))
    want = layer.output_proj(routed + shared + x2, ctx).reshape(x.shape)
    assert torch.allclose(y, want, atol=1e-5)


def test_shared_expert_layer_trains_every_parameter_and_reports_balance():
    cfg = SharedExpertConfig(16, 1, 4, 24, top_k=2)
    layer = SharedExpertLayer.new(BE, cfg)
    x = torch.randn(64, 16, generator=torch.Generator().manual_seed(1))
    out = layer(x, ForwardCtx.train(BE))
    (out.square().mean() + layer.last_aux_loss).backward()
    assert all(p.tensor.grad is not None and torch.isfinite(p.tensor.grad).all() for p in layer.parameters())
    names = [n for n, _ in layer.named_parameters()]
    assert {"router", "routed_w1", "routed_w2", "output_proj.weight", "shared_experts.0.gate_up.weight"} <= set(names)
    st = layer.stats(x)
    assert sum(st.tokens_per_routed_expert) == 64 * 2 and 0 < st.load_balance_score <= 1.0
    assert st.load_balance_score == pytest.approx((128 / 4) / max(st.tokens_per_routed_expert))
    assert SharedAndRoutedConfig(shared=2, routed=64, active_routed=6).active_fraction() == pytest.approx(8 / 66)


# ---- sampler --------------------------------------------------------------------------------------------------------
def test_sampler_greedy_top_k_nucleus_and_seed():
    logits = torch.tensor([[2.0, 1.0, 0.5, -1.0, -3.0]]).repeat(400, 1)
    assert Sampler.greedy().sample(logits).tolist() == [0] * 400
    top2 = Sampler(temperature=1.0, top_k=2, seed=1).sample(logits)
    assert set(top2.tolist()) == {0, 1}
    frac0 = float((top2 == 0).float().mean())
    assert abs(frac0 - float(torch.softmax(torch.tensor([2.0, 1.0]), 0)[0])) < 0.08          # 0.731 within sampling noise
    p = torch.softmax(logits[0], 0)                     # 0.609 0.224 0.136 0.030 0.004: nucleus 0.8 keeps the first two
    nucleus = Sampler(temperature=1.0, top_p=0.8, seed=2).sample(logits)
    assert set(nucleus.tolist()) == {0, 1} and float(p[:2].sum()) > 0.8 > float(p[0])
    everything = Sampler(temperature=1.0, seed=3).sample(logits)
    assert len(set(everything.tolist())) >= 4
    cold = Sampler(temperature=0.05, seed=4).sample(logits)
    assert (cold == 0).float().mean() > 0.99            # low temperature approaches the arg-max
    a, b = Sampler(1.0, seed=9).sample(logits), Sampler(1.0, seed=9).sample(logits)
    assert torch.equal(a, b) and not torch.equal(a, Sampler(1.0, seed=10).sample(logits))


# ---- model registry -------------------------------------------------------------------------------------------------
def test_model_registry_entries_point_at_presets_that_exist():
    from rustral_b200.models.config import preset
    from rustral_b200.utils.model_zoo import registry
    reg = registry()
    assert reg.schema_version == "1.0" and [e.id for e in reg.entries] == ["tiny-lm", "gpt2-small", "llama-8b", "moe-8x"]
    assert reg.get("nope") is None and reg.get("gpt2-small").huggingface_model_id == "openai-community/gpt2"
    g = preset("gpt2-small")
    assert (g.n_layer, g.d_model, g.n_head) == (12, 768, 12)          # what the entry's notes promise
    l = preset("llama-8b")
    assert (l.n_layer, l.d_model, l.n_head, l.n_kv_head) == (32, 4096, 32, 8)


# ---- metrics event file ---------------------------------------------------------------------------------------------
def test_event_file_gets_the_training_summary_and_histograms(tmp_path):
    from rustral_b200.metrics import MetricsLogger, TensorBoardWriter
    w = TensorBoardWriter(str(tmp_path), "run1")
    log = MetricsLogger([w])
    log.log_training_summary(3, 0.25, accuracy=0.9, lr=1e-3)
    log.set_step(7)
    log.log_scalar("grad_norm", 1.5)
    log.log_histogram("weights", [0.0, 0.1, 0.1, 0.9], bins=3)
    log.flush()
    rows = [json.loads(l) for l in open(tmp_path / "run1.jsonl")]
    assert [(r["type"], r["name"], r["step"]) for r in rows] == [("scalar", "train/loss", 3), ("scalar", "train/accuracy", 3),
                                                                  ("scalar", "train/lr", 3), ("scalar", "grad_norm", 7), ("histogram", "weights", 7)]
    assert rows[0]["value"] == 0.25 and rows[4]["counts"] == [3, 0, 1] and len(rows[4]["edges"]) == 4
    assert all(r["timestamp"] > 1e9 for r in rows)


# ---- tensor pool and memory profiler --------------------------------------------------------------------------------
def test_tensor_pool_reuses_released_buffers_by_shape_and_respects_its_limits():
    pool = TensorPool(PoolStrategy.STANDARD, max_per_shape=2, max_total=3)
    a = pool.acquire((16, 16))
    ptr = a.data_ptr()
    pool.release(a)
    b = pool.acquire((16, 16))
    assert b.data_ptr() == ptr and pool.stats()["hits"] == 1 and pool.stats()["misses"] == 1
    c = pool.acquire((16, 16), torch.float64)                           # another dtype is another bucket
    assert c.dtype == torch.float64 and c.data_ptr() != ptr
    for t in [b, c, pool.acquire((16, 16)), pool.acquire((16, 16)), pool.acquire((20, 20))]:
        pool.release(t)
    assert pool.total_free() == 3                                        # max_total caps what is kept
    tiny = pool.acquire((2, 2))
    pool.release(tiny)
    assert pool.total_free() == 3                                        # below min_elems: never pooled
    pool.clear()
    assert pool.total_free() == 0
    arena = TensorPool(PoolStrategy.TRAINING_ARENA)
    t1 = arena.acquire((8, 8))
    assert arena.total_free() == 0
    arena.begin_step()                                                   # everything lent in the step comes back at once
    assert arena.total_free() == 1 and arena.acquire((8, 8)).data_ptr() == t1.data_ptr()


def test_memory_profiler_tracks_peaks_leaks_and_risk():
    mem = MemoryProfiler(capacity_bytes=1000)
    h1 = mem.alloc("weights", 400)
    with mem.track_tensor("activations", torch.zeros(50)):              # 200 bytes
        snap = mem.snapshot("inside")
        assert snap["current"] == 600 and snap["by_tag"] == {"weights": 400, "activations": 200}
    after = mem.snapshot("after")
    assert after["current"] == 400 and after["peak"] == 600 and [s["label"] for s in mem.snapshots] == ["inside", "after"]
    assert mem.predict_oom_risk(0) == "low" and mem.predict_oom_risk(200) == "medium"
    assert mem.predict_oom_risk(400) == "high" and mem.predict_oom_risk(580) == "critical"
    assert [(tag, n) for _, tag, n in mem.find_leaks(older_than_s=0.0)] == [("weights", 400)]
    assert mem.find_leaks(older_than_s=3600.0) == []
    mem.free(h1)
    mem.free(h1)                                                         # freeing twice is harmless
    assert mem.find_leaks() == [] and mem.snapshot()["current"] == 0
    events = json.loads(mem.export_timeline())
    assert [e["kind"] for e in events] == ["alloc", "alloc", "free", "free"]


@pytest.mark.skipif(__import__("os").environ.get("RUSTRAL_TEST_HF_NETWORK") != "1",
                    reason="network smoke test of the hub loader: set RUSTRAL_TEST_HF_NETWORK=1 (crates/hf/src/lib.rs:219)")
def test_hub_download_smoke():
    from rustral_b200.utils.hf import download_state_dict
    state = download_state_dict("hf-internal-testing/tiny-random-gpt2")
    assert state and all(v.dtype == torch.float32 for v in state.values())
