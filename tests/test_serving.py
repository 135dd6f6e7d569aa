"""Serving stack on the CPU reference path: caches, scheduler, engine (paged decode == full re-forward), HTTP."""
import json
import urllib.request

import pytest
import torch

from rustral_b200.models.config import preset
from rustral_b200.runtime.fused_gpt import FusedGPTEngine
from rustral_b200.serve import (CacheConfig, KVCache, ModelRunner, PagedCache, RequestPriority, Sampler, Scheduler,
                                SchedulingPolicy, ServingEngine, SlidingWindowCache, run_poisson_workload)


def test_kv_cache_append_stores_values_and_rejects_overflow():
    c = KVCache(CacheConfig(num_heads=4, head_dim=8, max_seq_len=6).with_gqa(2))
    k, v = torch.randn(1, 2, 4, 8), torch.randn(1, 2, 4, 8)
    c.append(k, v)
    kk, vv = c.get()
    assert kk.shape == (1, 2, 4, 8) and torch.allclose(kk.float(), k, atol=1e-2) and torch.allclose(vv.float(), v, atol=1e-2)
    with pytest.raises(Exception):
        c.append(torch.randn(1, 2, 3, 8), torch.randn(1, 2, 3, 8))
    assert CacheConfig(32, 128, 4096, num_layers=32).with_gqa(8).memory_bytes() == 2 * 8 * 4096 * 128 * 32 * 2


def test_sliding_window_keeps_last_entries_in_order():
    c = SlidingWindowCache(CacheConfig(1, 2, 100), window=3)
    for i in range(5):
        c.append(torch.full((1, 1, 1, 2), float(i)), torch.full((1, 1, 1, 2), float(i)))
    k, _ = c.get()
    assert k[0, 0, :, 0].float().tolist() == [2.0, 3.0, 4.0]


def test_paged_cache_second_allocate_extends_table():
    pc = PagedCache(8, 16, allocate_storage=False)
    assert pc.allocate(7, 20) and pc.block_table(7) == [0, 1]
    assert pc.allocate(7, 40) and pc.block_table(7) == [0, 1, 2]       # extended, not overwritten
    assert pc.slot(7, 33) == 2 * 16 + 1
    assert not pc.allocate(9, 16 * 6) and pc.free_blocks == 5          # refused, nothing leaked
    assert pc.free(7) == 3 and pc.free_blocks == 8 and pc.block_table(7) == []


def test_scheduler_admission_policy_and_memory_pressure():
    pc = PagedCache(4, 16, allocate_storage=False)
    s = Scheduler(pc, max_batch_size=8, policy=SchedulingPolicy.PRIORITY)
    a = s.add_request(list(range(20)), 4, RequestPriority.LOW)
    b = s.add_request(list(range(20)), 4, RequestPriority.HIGH)
    c = s.add_request(list(range(40)), 4, RequestPriority.LOW)        # does not fit while a and b run
    batch = s.schedule()
    assert batch.request_ids == [b, a] and all(batch.is_prefill)
    s.update({a: 5, b: 6})
    batch = s.schedule()
    assert batch.input_ids == [[6], [5]] and not any(batch.is_prefill)
    for _ in range(3):
        s.update({a: 1, b: 1})
        batch = s.schedule()
    assert s.stats.completed == 2 and batch.request_ids == [c]
    assert pc.free_blocks == 4 - 3


def test_engine_paged_decode_matches_full_reforward():
    for name in ("gpt2-test", "llama-test"):
        cfg = preset(name, seq_len=64, d_model=64, ffn_dim=128)
        runner = ModelRunner(cfg, device="cpu", num_blocks=32)
        eng = ServingEngine(runner, max_batch_size=4)
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 17, 9)]
        ids = [eng.submit(p, 5) for p in prompts]
        eng.run_to_completion()
        ref = FusedGPTEngine(cfg, "cpu")
        ref.params = runner.params
        for p, rid in zip(prompts, ids):
            toks = list(p)
            for _ in range(5):
                pad = toks + [0] * (cfg.seq_len - len(toks))
                toks.append(int(ref.logits(torch.tensor([pad]))[0, len(toks) - 1].argmax()))
            assert eng.scheduler.get(rid).generated == toks[len(p):]
        assert runner.cache.free_blocks == 32
        m = eng.metrics(1.0)
        assert m.completed == 3 and m.output_tokens == 15 and m.ttft_p50_ms >= 0


def test_poisson_workload_and_sampler():
    cfg = preset("gpt2-test", seq_len=64, d_model=64, ffn_dim=128)
    eng = ServingEngine(ModelRunner(cfg, device="cpu", num_blocks=64), max_batch_size=8)
    m = run_poisson_workload(eng, 6, rate_per_s=200.0, prompt_range=(4, 12), output_range=(2, 4), seed=1)
    assert m.completed == 6 and m.output_tokens >= 12 and m.output_tokens_per_s > 0
    s = Sampler(temperature=1.0, top_k=5, top_p=0.9, seed=3)
    logits = torch.randn(4, 50)
    t = s.sample(logits)
    top5 = logits.topk(5, -1).indices
    assert all(int(t[i]) in top5[i].tolist() for i in range(4))
    assert Sampler.greedy().sample(logits).tolist() == logits.argmax(-1).tolist()


def test_http_server_routes_and_validation(tmp_path):
    from rustral_b200.core import CpuBackend
    from rustral_b200.nn.linear import LinearBuilder
    from rustral_b200.runtime.model_io import load_model_from_path, save_model_to_path
    from rustral_b200.serve.http_server import ServerState, linear_infer_fn, start_background
    b = CpuBackend()
    lin = LinearBuilder(4, 3).with_bias().build(b)
    path = str(tmp_path / "lin.safetensors")
    save_model_to_path(lin, path)
    lin2 = LinearBuilder(4, 3).with_bias().seed(9).build(b)
    load_model_from_path(lin2, path)
    state = ServerState(linear_infer_fn(lin2, 4), metadata={"model": "linear"})
    httpd, _ = start_background(state)
    base = f"http://127.0.0.1:{httpd.server_address[1]}"
    try:
        assert json.load(urllib.request.urlopen(base + "/health"))["status"] == "ok"
        assert json.load(urllib.request.urlopen(base + "/v1/metadata"))["model"] == "linear"
        req = urllib.request.Request(base + "/v1/infer", json.dumps({"input": [[1, 2, 3, 4]]}).encode(),
                                     {"Content-Type": "application/json"})
        out = json.load(urllib.request.urlopen(req))["output"]
        want = lin(torch.tensor([[1., 2., 3., 4.]])).tolist()
        assert torch.allclose(torch.tensor(out), torch.tensor(want), atol=1e-5)
        for bad in ({"input": []}, {"input": [[1, 2]]}):
            req = urllib.request.Request(base + "/v1/infer", json.dumps(bad).encode())
            with pytest.raises(urllib.error.HTTPError) as e:
                urllib.request.urlopen(req)
            assert e.value.code == 400
        text = urllib.request.urlopen(base + "/metrics").read().decode()
        assert "rustral_infer_requests_total 3" in text and "rustral_infer_errors_total 2" in text
    finally:
        httpd.shutdown()
        state.shutdown()


@pytest.mark.parametrize("policy", ["FCFS", "SRTF", "PRIORITY"])
def test_native_scheduler_core_makes_the_same_decisions_as_the_python_specification(policy):
    """Random arrivals, priorities, lengths and end-of-sequence hits on a cache small enough to force head-of-line
    blocking, preemption and pause-on-update: batch for batch the C++ core and the Python scheduler agree."""
    import random
    from rustral_b200.serve.kv_cache import PagedCache
    from rustral_b200.serve.scheduler import PyScheduler, RequestPriority, Scheduler, SchedulingPolicy
    for seed in range(6):
        rng = random.Random(seed)
        caches = [PagedCache(num_blocks=24, block_size=4, allocate_storage=False) for _ in range(2)]
        kw = dict(max_batch_size=5, policy=SchedulingPolicy[policy], preemption_threshold=0.5, max_prefill_tokens=40)
        a, b = PyScheduler(caches[0], **kw), Scheduler(caches[1], **kw)
        step, submitted = 0, 0
        while step < 400 and (submitted < 40 or a.has_work()):
            if submitted < 40 and rng.random() < 0.5:
                prompt = [rng.randrange(3, 50) for _ in range(rng.randrange(1, 30))]
                args = (prompt, rng.randrange(1, 12), RequestPriority(rng.randrange(0, 4)), 7 if rng.random() < 0.5 else None)
                assert a.add_request(*args) == b.add_request(*args)
                submitted += 1
            ba, bb = a.schedule(), b.schedule()
            assert (ba.request_ids, ba.input_ids, ba.seq_lens, ba.is_prefill) == (bb.request_ids, bb.input_ids, bb.seq_lens, bb.is_prefill)
            assert ba.block_tables == bb.block_tables
            assert a.has_work() == b.has_work() and caches[0].free_blocks == caches[1].free_blocks
            outs = {rid: (7 if rng.random() < 0.1 else rng.randrange(8, 50)) for rid in ba.request_ids}
            a.update(outs, now=float(step))
            b.update(outs, now=float(step))
            assert [r.id for r in a.paused] == [r.id for r in b.paused] and list(a.running) == list(b.running)
            assert [r.id for r in a.pending] == [r.id for r in b.pending]
            step += 1
        a._retire()
        b._retire()
        sa, sb = a.stats, b.stats
        assert (sa.completed, sa.preempted, sa.admitted, sa.total_generated) == (sb.completed, sb.preempted, sb.admitted, sb.total_generated)
        assert [(r.id, r.generated) for r in a.completed] == [(r.id, r.generated) for r in b.completed]
        assert sa.completed == 40 and not a.has_work() and caches[1].free_blocks == 24
        assert all(b.get(r.id).state.value == "completed" for r in b.completed)
        b.forget(b.completed[0].id)
        assert b.get(b.completed[0].id) is None


def test_generate_releases_the_request_record():
    """A server that answers through `generate` does not accumulate finished requests, in Python or in the native core."""
    cfg = preset("gpt2-test", seq_len=64, d_model=64, ffn_dim=128)
    eng = ServingEngine(ModelRunner(cfg, device="cpu", num_blocks=32), max_batch_size=4)
    for i in range(5):
        toks = eng.generate([3, 4, 5 + i], 3)
        assert len(toks) == 3
    sch = eng.scheduler
    assert sch.completed == [] and sch.requests == {} and not sch.has_work() and sch.stats.completed == 5
    kept = eng.generate([7, 8], 2, keep_record=True)
    assert len(sch.completed) == 1 and sch.completed[0].generated == kept
    rid = sch.completed[0].id
    eng.release(rid)
    eng.release(rid)                                  # idempotent
    assert sch.completed == [] and sch.get(rid) is None
    pending = eng.submit([1, 2, 3], 2)
    eng.release(pending)                              # not completed: left alone
    assert sch.get(pending) is not None


def test_http_server_decoder_engine_mode_and_inference_weight_loading(tmp_path):
    """`--model` builds the continuous-batching engine behind /v1/generate, with weights loaded strictly from a
    checkpoint in the trainer's format; the served tokens are the engine's own greedy tokens."""
    from rustral_b200.core.errors import SerializationError
    from rustral_b200.io import safetensors_io as st
    from rustral_b200.serve.http_server import build_state, parse_args, start_background
    from rustral_b200.serve.weights import InferenceWeights
    cfg = preset("llama-test", seq_len=64, d_model=64, ffn_dim=128)
    donor = ModelRunner(cfg, device="cpu", num_blocks=16, seed=5)
    path = str(tmp_path / "m.safetensors")
    st.save_file(donor.params.state_dict(), path)
    args = ["--model", "llama-test", "--weights", path, "--blocks", "32", "--max-batch", "4", "--seed", "1"]
    import rustral_b200.models.config as C
    saved = dict(C.PRESETS["llama-test"])
    C.PRESETS["llama-test"].update(seq_len=64, d_model=64, ffn_dim=128)
    try:
        state = build_state(parse_args(args))
    finally:
        C.PRESETS["llama-test"].clear()
        C.PRESETS["llama-test"].update(saved)
    httpd, _ = start_background(state)
    base = f"http://127.0.0.1:{httpd.server_address[1]}"
    try:
        meta = json.load(urllib.request.urlopen(base + "/v1/metadata"))
        assert meta["model"] == "llama-test" and meta["weights"] == path and meta["kv_blocks"] == 32
        req = urllib.request.Request(base + "/v1/generate", json.dumps({"prompt": [5, 6, 7, 8], "max_tokens": 6}).encode())
        served = json.load(urllib.request.urlopen(req))["tokens"]
        want = ServingEngine(donor, max_batch_size=2).generate([5, 6, 7, 8], 6)
        assert served == want and len(served) == 6
        bad = urllib.request.Request(base + "/v1/generate", json.dumps({"prompt": [10 ** 9]}).encode())
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(bad)
        assert e.value.code == 400
    finally:
        httpd.shutdown()
        state.shutdown()
    # the bf16 inference weight set loads the same checkpoint strictly
    iw = InferenceWeights.random_llama(cfg, "cpu", seed=9)
    sd = donor.params.state_dict()
    iw.load_state_dict(sd, cfg)
    hd = cfg.head_dim
    assert torch.equal(iw.w("layers.0.attn.wqkv.weight")[:cfg.n_head * hd], sd["layers.0.attn.wq.weight"])
    assert torch.equal(iw.w("tok_embed.embed")[:cfg.vocab_size], sd["tok_embed.embed"])
    with pytest.raises(SerializationError):
        iw.load_state_dict({k: v for k, v in sd.items() if k != "final_norm.weight"}, cfg)
    with pytest.raises(SerializationError):
        iw.load_state_dict(dict(sd, bogus=torch.zeros(1)), cfg)
    with pytest.raises(SystemExit):
        build_state(parse_args([]))


def test_engine_loop_batches_concurrent_http_style_requests():
    """Requests from several handler threads join one running batch: same tokens as one-at-a-time generation, far
    fewer engine steps than the sum of the individual generations, records released afterwards."""
    import threading
    from rustral_b200.serve.http_server import EngineLoop
    cfg = preset("gpt2-test", seq_len=64, d_model=64, ffn_dim=128)
    runner = ModelRunner(cfg, device="cpu", num_blocks=64, seed=2)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 9, 3, 12, 7, 4)]
    solo = ServingEngine(ModelRunner(cfg, device="cpu", num_blocks=64, seed=2), max_batch_size=8)
    want = [solo.generate(p, 10) for p in prompts]
    eng = ServingEngine(runner, max_batch_size=8)
    loop = EngineLoop(eng)
    got, errs = [None] * len(prompts), []

    def worker(i):
        try:
            got[i] = loop.generate(prompts[i], 10, timeout=120)
        except Exception as e:      # noqa: BLE001
            errs.append(e)
    threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(prompts))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=180)
    try:
        assert not errs and got == want
        assert loop.steps < 6 * 10                      # 60 steps one after another; batched: little more than 10
        assert eng.scheduler.requests == {} and eng.scheduler.completed == [] and runner.cache.free_blocks == 64
        with pytest.raises(ValueError):
            loop.generate([], 3, timeout=10)            # the engine's own validation reaches the caller
        assert loop.generate(prompts[0], 10, timeout=60) == want[0]     # and the loop is still alive
    finally:
        loop.shutdown()


def test_paged_serving_engine_generates_the_tokens_hugging_face_generates():
    """Independent oracle for the whole serving path (paged KV cache, prefill + decode, continuous batching): greedy
    tokens equal `transformers` greedy generation for a GPT-2 and a Llama model; a model trained here exports back."""
    transformers = pytest.importorskip("transformers")
    from rustral_b200.utils.hf import config_from_hf, convert_hf_gpt2, convert_hf_llama, export_hf_gpt2
    torch.manual_seed(0)
    hc = transformers.GPT2Config(vocab_size=200, n_positions=48, n_embd=64, n_layer=2, n_head=4, resid_pdrop=0.0,
                                 embd_pdrop=0.0, attn_pdrop=0.0)
    lc = transformers.LlamaConfig(vocab_size=200, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=48, rope_theta=10000.0,
                                  rms_norm_eps=1e-5, tie_word_embeddings=False, attention_dropout=0.0)
    prompts = [[5, 17, 3, 99, 42], [7, 7, 8], [150, 2, 31, 64, 11, 9, 120]]
    for hf_cfg, cls, conv in ((hc, transformers.GPT2LMHeadModel, convert_hf_gpt2), (lc, transformers.LlamaForCausalLM, convert_hf_llama)):
        model = cls(hf_cfg).eval()
        cfg = config_from_hf(hf_cfg)
        runner = ModelRunner(cfg, device="cpu", num_blocks=32)
        runner.params.load_state_dict(conv(model.state_dict()))
        eng = ServingEngine(runner, max_batch_size=4)
        ids = [eng.submit(p, 10) for p in prompts]                  # all three in one continuous batch
        eng.run_to_completion()
        for p, rid in zip(prompts, ids):
            with torch.no_grad():
                ref = model.generate(torch.tensor([p]), max_new_tokens=10, do_sample=False, pad_token_id=0)[0, len(p):].tolist()
            assert eng.scheduler.get(rid).generated == ref, (cfg.arch, p)
        if cfg.arch == "gpt2":
            back = export_hf_gpt2(runner.params.state_dict())
            ref_sd = {k: v for k, v in model.state_dict().items() if not k.endswith((".attn.bias", ".attn.masked_bias"))}
            assert set(back) == set(ref_sd) and all(torch.allclose(back[k], ref_sd[k].float(), atol=1e-7) for k in ref_sd)


@pytest.mark.parametrize("name", ["gpt2-test", "llama-test"])
def test_chunked_and_batched_prefill_generate_the_same_tokens_as_whole_prompt_prefill(name):
    """Prompts cut into chunks of 4 or 7 tokens that share their model pass with other prompts' chunks and with the decode
    batch (the later chunks attend to keys gathered from the pages) give the tokens of one-prompt-at-a-time prefill."""
    cfg = preset(name, seq_len=64, d_model=64, ffn_dim=128)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 23, 9, 1, 16)]
    results, steps = {}, {}
    for chunk in (0, 4, 7, 2048):
        runner = ModelRunner(cfg, device="cpu", num_blocks=32, block_size=4)
        eng = ServingEngine(runner, max_batch_size=4, prefill_chunk=chunk)
        ids = [eng.submit(p, 6) for p in prompts[:3]]
        eng.step()                                     # the remaining requests arrive while the first are being served
        ids += [eng.submit(p, 6) for p in prompts[3:]]
        eng.run_to_completion()
        results[chunk] = [eng.scheduler.get(r).generated for r in ids]
        steps[chunk] = eng.steps
        assert runner.cache.free_blocks == 32 and not eng._prefill_pos
    assert results[4] == results[0] and results[7] == results[0] and results[2048] == results[0]
    assert steps[4] > steps[2048]                      # small chunks spread the 23-token prompt over several steps


def test_a_long_prompt_does_not_stall_running_requests_for_more_than_a_chunk():
    cfg = preset("gpt2-test", seq_len=64, d_model=64, ffn_dim=128)
    eng = ServingEngine(ModelRunner(cfg, device="cpu", num_blocks=32, block_size=4), max_batch_size=4, prefill_chunk=8)
    a = eng.submit([1, 2, 3], 12)
    eng.step()                                         # request a is decoding now
    b = eng.submit(list(range(1, 41)), 2)              # 40-token prompt: five chunks
    produced = []
    for _ in range(5):
        out = eng.step()
        produced.append((a in out, b in out))
    assert produced == [(True, False)] * 4 + [(True, True)]


def test_serving_benchmark_rate_sweep_stops_at_saturation(capsys):
    """The sweep reports one row per rate, the capacity, and stops after the first rate whose p99 TTFT exceeds the limit."""
    import json
    from rustral_b200.serve import bench_serving
    bench_serving.main(["--model", "gpt2-test", "--requests", "5", "--rates", "400", "100", "200", "--prompt", "4", "10",
                        "--output", "2", "3", "--blocks", "64", "--ttft-limit-ms", "1e9", "--prefill-chunk", "6"])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert [r["rate_per_s"] for r in out["sweep"]] == [100.0, 200.0, 400.0] and out["saturated_at_rate"] is None
    assert all(r["completed"] == 5 for r in out["sweep"]) and out["prefill_chunk"] == 6
    assert out["capacity_tokens_per_s"] == max(r["output_tokens_per_s"] for r in out["sweep"])
    bench_serving.main(["--model", "gpt2-test", "--requests", "4", "--rates", "50", "100", "--prompt", "4", "10", "--output", "2", "3",
                        "--blocks", "64", "--ttft-limit-ms", "0"])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert len(out["sweep"]) == 1 and out["saturated_at_rate"] == 50.0


@pytest.mark.parametrize("chunk", [0, 5])
def test_a_cache_too_small_for_all_requests_pauses_and_resumes_without_changing_any_output(chunk):
    """Twelve requests through a cache that holds about four of them: requests are paused when a step cannot get a block,
    their blocks are released, and they are recomputed from their tokens on resume.  With greedy sampling the generated
    tokens must equal those of an engine with room for everything, whole-prompt or chunked prefill alike."""
    cfg = preset("llama-test", seq_len=64, d_model=64, ffn_dim=128)
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist() for n in torch.randint(2, 14, (12,), generator=g)]
    outs = {}
    for blocks in (64, 20):
        runner = ModelRunner(cfg, device="cpu", num_blocks=blocks, block_size=4, seed=1)
        eng = ServingEngine(runner, max_batch_size=6, prefill_chunk=chunk)
        ids = []
        for i, p in enumerate(prompts):                # arrivals are spread over the first steps
            ids.append(eng.submit(p, 10))
            if i % 3 == 2:
                eng.step()
        eng.run_to_completion(max_steps=2000)
        outs[blocks] = [eng.scheduler.get(r).generated for r in ids]
        assert all(len(o) == 10 for o in outs[blocks]) and runner.cache.free_blocks == blocks and not eng._prefill_pos
        if blocks == 20:
            assert eng.scheduler.stats.preempted > 0    # the small cache really did run out
    assert outs[20] == outs[64]


def test_aborting_a_request_frees_its_blocks_and_leaves_the_others_untouched():
    cfg = preset("gpt2-test", seq_len=64, d_model=64, ffn_dim=128)
    prompts = [[5, 6, 7, 8, 9], [11, 12, 13], [21, 22, 23, 24, 25, 26, 27]]

    def run(abort_second: bool):
        runner = ModelRunner(cfg, device="cpu", num_blocks=32, block_size=4, seed=2)
        eng = ServingEngine(runner, max_batch_size=4)
        ids = [eng.submit(p, 8) for p in prompts]
        eng.step(); eng.step()
        if abort_second:
            used = runner.cache.free_blocks
            assert eng.abort(ids[1]) and runner.cache.free_blocks > used
            assert not eng.abort(ids[1]) and not eng.abort(999)
        eng.run_to_completion()
        assert runner.cache.free_blocks == 32
        return [eng.scheduler.get(r).generated if eng.scheduler.get(r) is not None else None for r in ids]
    full, cut = run(False), run(True)
    assert cut[0] == full[0] and cut[2] == full[2] and len(full[1]) == 8
    assert cut[1] is None or len(cut[1]) < 8


def test_aborting_during_chunked_prefill_drops_the_prefill_progress():
    cfg = preset("gpt2-test", seq_len=64, d_model=64, ffn_dim=128)
    eng = ServingEngine(ModelRunner(cfg, device="cpu", num_blocks=32, block_size=4), max_batch_size=4, prefill_chunk=4)
    rid = eng.submit(list(range(1, 30)), 3)
    eng.step()
    assert eng._prefill_pos.get(rid) == 4                    # one chunk of the 29-token prompt is in the cache
    assert eng.abort(rid) and rid not in eng._prefill_pos and eng.runner.cache.free_blocks == 32
    other = eng.submit([3, 4, 5], 2)
    eng.run_to_completion()
    assert len(eng.scheduler.get(other).generated) == 2
    eng2 = ServingEngine(ModelRunner(cfg, device="cpu", num_blocks=32, block_size=4), max_batch_size=4, prefill_chunk=4)
    a = eng2.submit(list(range(1, 30)), 3)
    eng2.step()
    assert eng2.abort_all() == [a] and not eng2._prefill_pos and not eng2.scheduler.has_work()
