"""End-to-end smoke of the CPU tiny-LM example (config: 2 layers, d128, vocab 1024, seq 64, batch 8, Adam 1e-3)."""
import importlib.util
import json
import os

import pytest


def test_tiny_lm_cpu_trains_and_roundtrips(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("tiny_lm_cpu", os.path.join(root, "examples", "tiny_lm_cpu.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    m = mod.main(["--steps", "12", "--out", str(tmp_path)])
    assert m["loss_end"] < m["loss_start"] - 0.3 and m["checkpoint_roundtrip_ok"]
    assert abs(m["loss_start"] - 6.93) < 0.2                      # ln(1024) at initialisation
    assert json.load(open(tmp_path / "manifest.json"))["steps"] == 12
    assert (tmp_path / "model.safetensors").exists() and (tmp_path / "tiny_lm.jsonl").exists()


def _load_example(name):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location(name, os.path.join(root, "examples", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_SST2_TSV = ("sentence\tlabel\nthis movie was great\t1\nawful boring waste of time\t0\n"
             "the acting was wonderful and inspired\t1\ncompletely terrible\t0\nfun and exciting and amazing\t1\n"
             "bad bad bad really bad\t0\nlovely and heartwarming\t1\nawful again ugh\t0\n"
             "brilliant performance throughout\t1\ndisappointing ending\t0\n")


def _stage_sst2(tmp_path, monkeypatch, reps=1):
    d = tmp_path / "cache" / "datasets" / "sst2"
    d.mkdir(parents=True)
    body = _SST2_TSV + "".join(_SST2_TSV.split("\n", 1)[1] for _ in range(reps - 1))
    (d / "train.tsv").write_text(body)
    (d / "dev.tsv").write_text(_SST2_TSV)
    monkeypatch.setenv("RUSTRAL_CACHE_DIR", str(tmp_path / "cache"))
    monkeypatch.setenv("RUSTRAL_DATASET_OFFLINE", "1")
    monkeypatch.setenv("RUSTRAL_DATASET_SKIP_CHECKSUM", "1")


def test_sst2_classifier_runs_offline_quick(tmp_path, monkeypatch):
    """The pre-staged tiny corpus, `--quick`, and a well-formed manifest (crates/runtime/tests/sst2_smoke.rs)."""
    from rustral_b200.bench.manifest import validate_manifest
    _stage_sst2(tmp_path, monkeypatch)
    out = tmp_path / "out"
    _load_example("sst2_classifier").main(["--quick", "--out-dir", str(out)])
    m = json.load(open(out / "manifest.json"))
    assert m["task"] == "sst2_classifier" and m["quick_mode"] and "dev_accuracy" in m and "git_sha" in m
    assert m["vocab_size"] > 4 and m["train_examples"] == 10 and len(m["dataset_hash_fnv1a"]) == 16
    assert m["diagnostics"]["dev_label_counts"] == [5, 5] and sum(m["diagnostics"]["dev_positive_prob_hist"]) == 10
    assert validate_manifest(m) == [] and (out / "vocab.txt").read_text().startswith("<pad>\n<unk>\n<bos>\n<eos>\n")


def test_sst2_classifier_overfits_small_set(tmp_path, monkeypatch):
    """Training works end to end: the first 32 examples are memorised (crates/runtime/tests/sst2_overfit.rs)."""
    _stage_sst2(tmp_path, monkeypatch, reps=4)
    m = _load_example("sst2_classifier").main(["--overfit-32", "--epochs", "30", "--batch", "8", "--out-dir", str(tmp_path / "o")])
    assert m["overfit_32"] and m["dev_accuracy"] >= 0.95, m["dev_accuracy"]
    assert m["diagnostics"]["epoch_losses"][-1] < 0.5 * m["diagnostics"]["epoch_losses"][0]


def _stage_wikitext(tmp_path, monkeypatch):
    d = tmp_path / "cache" / "datasets" / "wikitext-2"
    d.mkdir(parents=True)
    words = "the of and in to a was is for as on with by that it from at his an were are which this be".split()
    text = "\n".join(" ".join(words[(i * 7 + j * (3 + i % 5)) % len(words)] for j in range(12)) + " ." for i in range(120))
    for s in ("train", "valid", "test"):
        (d / f"{s}.txt").write_text(text)
    monkeypatch.setenv("RUSTRAL_CACHE_DIR", str(tmp_path / "cache"))
    monkeypatch.setenv("RUSTRAL_DATASET_OFFLINE", "1")


def test_wikitext2_lm_runs_offline_quick(tmp_path, monkeypatch):
    """crates/runtime/tests/wikitext2_lm_smoke.rs: offline `--quick` run, manifest fields, vocabulary file."""
    from rustral_b200.bench.manifest import validate_manifest
    _stage_wikitext(tmp_path, monkeypatch)
    out = tmp_path / "out"
    m = _load_example("wikitext2_lm").main(["--quick", "--block-size", "16", "--d-model", "32", "--num-heads", "2",
                                            "--ffn-dim", "64", "--num-layers", "1", "--out-dir", str(out)])
    assert m["task"] == "wikitext2_word_lm" and m["dev_perplexity"] > 1.0 and m["vocab_size"] > 4
    assert m["dev_perplexity"] <= 1.2 * m["vocab_size"]            # no worse than uniform after one epoch
    assert validate_manifest(json.load(open(out / "manifest.json"))) == [] and (out / "vocab.txt").exists()


def test_wikitext2_lm_overfits_tiny(tmp_path, monkeypatch):
    """crates/runtime/tests/wikitext2_overfit.rs: eight windows are memorised."""
    _stage_wikitext(tmp_path, monkeypatch)
    m = _load_example("wikitext2_lm").main(["--overfit-tiny", "--block-size", "16", "--epochs", "60", "--batch", "8",
                                            "--out-dir", str(tmp_path / "o")])
    assert m["dev_perplexity"] < 2.0, m["dev_perplexity"]


def test_manifest_validation_and_curation(tmp_path):
    """scripts/bench/test_validate_manifest.py: missing keys and missing SST-2 diagnostics are reported."""
    from rustral_b200.bench import manifest as M
    good = M.write_manifest(str(tmp_path / "m.json"), "sst2_classifier", {
        "model_type": "transformer_encoder", "seed": 1, "total_params": 10, "vocab_size": 8, "epochs": 1, "batch_size": 2,
        "learning_rate": 1e-3, "dataset_hash_fnv1a": "0" * 16, "train_elapsed_sec": 0.1, "dataset": "d", "tokenizer": "t",
        "quick_mode": True, "dev_accuracy": 0.5, "dev_loss": float("nan")},
        {k: [] for k in M.SST2_DIAGNOSTICS})
    assert M.validate_manifest(good) == [] and good["dev_loss"] is None and "git_sha" in good
    bad = dict(good)
    del bad["seed"], bad["dev_accuracy"]
    bad["diagnostics"] = {}
    errs = M.validate_manifest(bad)
    assert len(errs) == 3 and any("seed" in e for e in errs) and any("diagnostics missing" in e for e in errs)
    cur = M.curate("sst2_classifier", "dev_accuracy", "v0", [dict(good, seed=s, dev_accuracy=a) for s, a in ((1, 0.5), (2, 0.7))])
    assert M.validate_curated(cur) == [] and abs(cur["aggregate"]["mean"] - 0.6) < 1e-9 and cur["aggregate"]["n"] == 2
    assert M.validate_curated({"runs": []})[-1].endswith("non-empty array")
    p = tmp_path / "c.json"
    p.write_text(json.dumps(cur))
    assert M.main([str(p), str(tmp_path / "m.json")]) == 0


def test_char_lm_trains_roundtrips_and_is_deterministic(tmp_path):
    """crates/runtime/examples/emnlp_char_lm.rs: loss falls, save / load keeps the logits, three runs agree."""
    mod = _load_example("emnlp_char_lm")
    r = mod.train_once(42, False)
    assert r["roundtrip_ok"] and r["epoch_losses"][-1] < 0.5 * r["epoch_losses"][0] and r["train_accuracy"] > 0.6
    assert r["generated"].startswith(mod.PROMPT) and len(r["generated"]) == len(mod.PROMPT) + mod.GENERATE_LEN
    rep = mod.main(["--determinism-check", "--out-dir", str(tmp_path)])
    assert rep["all_equal"] and json.load(open(tmp_path / "emnlp_determinism_report.json"))["all_equal"]


def test_nlp_eval_curates_multi_seed_runs(tmp_path, monkeypatch):
    """scripts/eval/run_nlp_real.py: per-seed manifests of both tasks under one curated file each."""
    from rustral_b200.bench import nlp_eval
    from rustral_b200.bench.manifest import validate_curated
    _stage_sst2(tmp_path, monkeypatch, reps=3)
    d = tmp_path / "cache" / "datasets" / "wikitext-2"
    d.mkdir(parents=True)
    words = "the of and in to a was is for as on with by that it from at his an were are which this be".split()
    text = "\n".join(" ".join(words[(i * 7 + j * (3 + i % 5)) % len(words)] for j in range(12)) + " ." for i in range(60))
    for s in ("train", "valid", "test"):
        (d / f"{s}.txt").write_text(text)
    out = tmp_path / "nlp"
    assert nlp_eval.main(["--benchmark", "--seeds", "0,1", "--out", str(out)]) == 0
    for task, metric in (("sst2", "dev_accuracy"), ("wikitext2", "dev_perplexity")):
        doc = json.load(open(out / f"{task}.json"))
        assert validate_curated(doc) == [] and doc["metric"] == metric and doc["aggregate"]["n"] == 2
        assert [r["seed"] for r in doc["runs"]] == [0, 1]
        assert (out / "raw" / task / "seed1" / "manifest.json").exists()
    seeds = json.load(open(out / "sst2.json"))["runs"]
    assert seeds[0]["manifest"]["vocab_size"] == seeds[1]["manifest"]["vocab_size"]


def test_pytorch_baselines_write_curated_manifests(tmp_path, monkeypatch):
    """benchmarks/pytorch/*_baseline.py: plain-PyTorch runs of both tasks end in `<task>_pytorch.json`."""
    from rustral_b200.bench import torch_baselines
    from rustral_b200.bench.manifest import validate_curated
    _stage_sst2(tmp_path, monkeypatch, reps=3)
    _stage_wikitext_into(tmp_path / "cache")
    out = tmp_path / "nlp"
    small = ["--seq-len", "16", "--d-model", "32", "--num-heads", "2", "--ffn-dim", "64", "--num-layers", "1", "--quick",
             "--seeds", "0,1", "--out", str(out)]
    assert torch_baselines.main(["--task", "sst2", *small]) == 0
    assert torch_baselines.main(["--task", "wikitext2", *small]) == 0
    for task, metric in (("sst2", "dev_accuracy"), ("wikitext2", "dev_perplexity")):
        doc = json.load(open(out / f"{task}_pytorch.json"))
        assert validate_curated(doc) == [] and doc["metric"] == metric and doc["aggregate"]["n"] == 2
        assert all(r["manifest"]["framework"] == "pytorch" for r in doc["runs"])
    assert json.load(open(out / "wikitext2_pytorch.json"))["runs"][0]["manifest"]["dev_perplexity"] > 1.0


def _stage_wikitext_into(cache):
    d = cache / "datasets" / "wikitext-2"
    d.mkdir(parents=True, exist_ok=True)
    words = "the of and in to a was is for as on with by that it from at his an were are which this be".split()
    text = "\n".join(" ".join(words[(i * 7 + j * (3 + i % 5)) % len(words)] for j in range(12)) + " ." for i in range(60))
    for s in ("train", "valid", "test"):
        (d / f"{s}.txt").write_text(text)


def test_bench_reference_arm_prints_one_json_line():
    """`bench.py --impl reference` answers with a single JSON line and exit code 0 even where the reference cannot run."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                          "--warmup", "3"], capture_output=True, text=True, timeout=120, cwd=root)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    doc = json.loads(lines[0])
    assert doc["impl"] == "reference" and (("unavailable" in doc and isinstance(doc["unavailable"], str) and "\n" not in doc["unavailable"])
                                           or "value" in doc)


def test_pretraining_example_checkpoints_asynchronously_and_resumes_exactly(tmp_path):
    """Token file -> prefetcher -> trainer -> asynchronous checkpoints; a run stopped at step 8 and resumed to 12
    reproduces the losses of the uninterrupted 12-step run."""
    mod = _load_example("pretrain_lm")
    common = ["--model", "gpt2-test", "--layers", "1", "--seq-len", "16", "--d-model", "32", "--global-batch", "4",
              "--micro-batch", "4", "--warmup", "2", "--checkpoint-every", "4", "--device", "cpu", "--lr", "3e-3"]
    full = mod.main([*common, "--steps", "12", "--out", str(tmp_path / "full")])
    assert full["loss_last"] < full["loss_first"] and full["last_checkpoint"] == 12
    for s in (4, 8, 12):
        d = tmp_path / "full" / f"step_{s}"
        assert (d / "model.safetensors").exists() and (d / "optimizer_rank_0.safetensors").exists() and (d / "complete.json").exists()
    part = mod.main([*common, "--steps", "12", "--stop-after", "8", "--out", str(tmp_path / "part")])
    assert part["losses"] == full["losses"][:8] and part["last_checkpoint"] == 8
    rest = mod.main([*common, "--steps", "12", "--out", str(tmp_path / "part"), "--resume"])
    assert rest["first_step"] == 8 and rest["losses"] == full["losses"][8:]
    assert json.load(open(tmp_path / "part" / "summary.json"))["last_checkpoint"] == 12


@pytest.mark.parametrize("layers", [0, 2])
def test_sst2_one_step_parity_against_plain_pytorch(tmp_path, monkeypatch, layers):
    """The example's one-step dump is reproduced by an independent torch.nn.functional model + torch.optim.Adam, and a
    tampered dump is caught (scripts/eval/sst2_parity_one_step.py)."""
    from rustral_b200.bench import sst2_parity
    _stage_sst2(tmp_path, monkeypatch, reps=2)
    dump = tmp_path / "parity.json"
    _load_example("sst2_classifier").main(["--overfit-32", "--num-layers", str(layers), "--parity-one-step", "--parity-batch", "8",
                                           "--parity-dump", str(dump), "--out-dir", str(tmp_path / "o")])
    doc = json.load(open(dump))
    assert len(doc["ids"]) == 8 and doc["config"]["num_layers"] == layers and set(doc["grads"]) == set(doc["params_before"])
    res = sst2_parity.check(doc)
    assert res["ok"], res
    assert res["logits"]["max_abs"] < 1e-5 and abs(res["loss"][0] - res["loss"][1]) < 1e-5
    head = [r for r in res["grads"] if r["name"] == "head.weight"][0]
    assert head["sign_agree"] == 1.0 and head["rel_l2"] < 1e-4 and head["norm_torch"] > 0
    assert sst2_parity.main([str(dump)]) == 0
    doc["grads"]["head.weight"] = [-g for g in doc["grads"]["head.weight"]]        # a sign error must be reported
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps(doc))
    assert sst2_parity.main([str(bad)]) == 1


def test_campaign_queue_runs_the_nlp_evaluation_its_twins_and_the_report(tmp_path, monkeypatch):
    """The one-shot job list: NLP evaluation of this framework, the plain-PyTorch twins on the same vocabulary, and the
    comparative report with both (scripts/bench/queue_all_benchmarks.sh with RUN_NLP_PAPER / RUN_NLP_PYTORCH)."""
    from rustral_b200.bench import reports
    _stage_sst2(tmp_path, monkeypatch, reps=3)
    _stage_wikitext_into(tmp_path / "cache")
    res = reports.run_queue(tmp_path / "bench", [], repeats=1, warmup=0, nlp="benchmark", seeds="0", device="cpu", strict=True)
    assert res["failures"] == 0, res["steps"]
    assert [n for n, _ in res["steps"]] == ["NLP evaluation (benchmark, seeds 0)", "PyTorch twin: sst2", "PyTorch twin: wikitext2", "comparative report"]
    text = open(res["report"]).read()
    assert "SST-2 classifier" in text and "WikiText-2" in text and "PyTorch" in text and "over 1 seed" in text
