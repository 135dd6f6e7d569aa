"""Report tooling around the benchmark harness documents (rustral_b200/bench/reports.py)."""
import json

import pytest

from rustral_b200.bench import Sample, samples_to_json, validate_schema
from rustral_b200.bench import reports as R


def _doc(suite, scale):
    samples = [Sample("matmul.128x128x128", "b", "cpu", "f32", None, {"m": 128}, [1.0 * scale, 1.2 * scale, 1.1 * scale]),
               Sample("softmax_dim.32x64", "b", "cpu", "f32", None, {"rows": 32}, [0.5 * scale, 0.5 * scale])]
    d = json.loads(samples_to_json(samples, suite=suite))
    assert validate_schema(d) == []
    return d


def test_combine_and_summary_speedup_column():
    ours, base = _doc("rustral-b200-cpu", 1.0), _doc("torch-cpu", 2.0)
    doc = R.combine([ours, base])
    assert doc["suites"] == ["rustral-b200-cpu", "torch-cpu"] and len(doc["samples"]) == 4
    md = R.summary_markdown(doc, "torch-cpu")
    row = [l for l in md.splitlines() if l.startswith("| matmul")][0]
    assert "2.00x" in row and "1.1000" in row and "2.2000" in row      # baseline mean / our mean
    assert "speed-up vs torch-cpu" in md.splitlines()[0]


def test_bmf_export_names_and_units():
    bmf = R.to_bmf(R.combine([_doc("suiteA", 1.0)]))
    k = "suiteA/b/cpu/matmul.128x128x128"
    assert k in bmf
    lat = bmf[k]["latency"]
    assert lat["lower_value"] == pytest.approx(1.0e6) and lat["upper_value"] == pytest.approx(1.2e6)
    assert lat["value"] == pytest.approx(1.1e6)


def test_index_regeneration_and_stale_check(tmp_path):
    for v, sha in (("v0.1.0", "a" * 40), ("v0.2.0", "b" * 40)):
        d = tmp_path / v
        d.mkdir()
        (d / "manifest.json").write_text(json.dumps({"version": v, "git_sha": sha, "date": "2026-01-01", "machine": "b200"}))
        (d / "cpu.json").write_text("{}")
    (tmp_path / "INDEX.md").write_text("# Snapshots\n\nhand-written introduction\n\n## Index\n\nold table\n")
    assert R.main(["index", "--runs-dir", str(tmp_path), "--check"]) == 1          # stale
    assert R.main(["index", "--runs-dir", str(tmp_path)]) == 0
    text = (tmp_path / "INDEX.md").read_text()
    assert "hand-written introduction" in text and "| v0.2.0 | 2026-01-01 | bbbbbbbbbbbb | b200 | cpu |" in text
    assert R.main(["index", "--runs-dir", str(tmp_path), "--check"]) == 0
    (tmp_path / "v0.2.0" / "manifest.json").write_text(json.dumps({"version": "v0.2.0"}))
    with pytest.raises(ValueError, match="missing keys"):
        R.index_table(tmp_path)


def test_compare_and_emnlp_reports(tmp_path):
    h = tmp_path / "h.json"
    h.write_text(json.dumps(R.combine([_doc("rustral-b200-cpu", 1.0), _doc("torch-cpu", 3.0)])))
    nlp = tmp_path / "runs" / "nlp"
    nlp.mkdir(parents=True)
    (nlp / "sst2.json").write_text(json.dumps({"runs": [{"accuracy": 0.5, "throughput": 100.0}, {"accuracy": 0.7, "throughput": 120.0}]}))
    (nlp / "sst2_pytorch.json").write_text(json.dumps({"runs": [{"accuracy": 0.6, "throughput": 80.0}]}))
    out = tmp_path / "cmp.md"
    assert R.main(["compare", "--harness", str(h), "--runs", str(tmp_path / "runs"), "--baseline", "torch-cpu", "--out", str(out)]) == 0
    text = out.read_text()
    assert "3.00x" in text and "accuracy 0.6000 +- 0.1414 over 2 seed(s)" in text and "PyTorch twin: accuracy 0.6000 over 1" in text
    assert "no curated file" in text                                    # the WikiText-2 files are absent
    out2 = tmp_path / "emnlp.md"
    assert R.main(["emnlp", "--harness", str(h), "--runs", str(tmp_path / "runs"), "--out", str(out2)]) == 0
    t2 = out2.read_text()
    assert "## Micro-benchmarks: torch-cpu" in t2 and "## Environment" in t2


def test_torch_suite_mirrors_the_framework_workload_names():
    import torch
    from rustral_b200.bench import workloads
    from rustral_b200.core import CpuBackend
    ours = {n for n, _, _ in workloads.build_workloads(CpuBackend())}
    twin = {n for n, _, _, _ in R._torch_workloads("cpu", heavy=False)}
    assert twin <= ours and len(twin) >= 17
    assert R.run_suite("torch-cuda", 1, 0) is None or torch.cuda.is_available()


def test_regression_gate_needs_both_a_slowdown_and_disjoint_intervals(tmp_path):
    base = _doc("s", 1.0)
    slow = _doc("s", 2.5)                                   # 2.5x slower, intervals far apart
    res = R.regress(base, slow, 1.15)
    assert [r["regression"] for r in res["rows"]] == [True, True] and res["rows"][0]["ratio"] == pytest.approx(2.5)
    noisy = json.loads(samples_to_json([Sample("matmul.128x128x128", "b", "cpu", "f32", None, {"m": 128}, [0.5, 2.5, 0.9]),
                                        Sample("other", "b", "cpu", "f32", None, {}, [1.0, 1.0])], suite="s"))
    res = R.regress(base, noisy, 1.15)                     # mean 1.3 vs 1.1 (x1.18) but the interval is wide: not a failure
    assert len(res["rows"]) == 1 and res["rows"][0]["ratio"] > 1.15 and not res["rows"][0]["regression"]
    assert [k[1] for k in res["missing"]] == ["softmax_dim.32x64"] and [k[1] for k in res["extra"]] == ["other"]
    b, c, n = tmp_path / "b.json", tmp_path / "c.json", tmp_path / "n.json"
    b.write_text(json.dumps(base)); c.write_text(json.dumps(slow)); n.write_text(json.dumps(noisy))
    assert R.main(["regress", "--baseline", str(b), "--current", str(c)]) == 0                     # report only
    assert R.main(["regress", "--baseline", str(b), "--current", str(c), "--fail-on-regression"]) == 1
    assert R.main(["regress", "--baseline", str(b), "--current", str(c), "--fail-on-regression", "--max-slowdown", "3.0"]) == 0
    assert R.main(["regress", "--baseline", str(b), "--current", str(n), "--fail-on-regression"]) == 0
    assert R.main(["regress", "--baseline", str(b), "--current", str(n), "--require-matching"]) == 1
    assert R.main(["regress", "--baseline", str(b), "--current", str(b), "--fail-on-regression", "--require-matching"]) == 0


def test_static_site_lists_snapshots_and_escapes_names(tmp_path):
    out = tmp_path / "site"
    assert [p.name for p in R.render_site(tmp_path / "absent", out)] == ["index.html"]
    assert "no snapshots yet" in (out / "index.html").read_text()
    runs = tmp_path / "runs"
    for v, scale in (("v0.1.0", 1.0), ("v0.2.0", 0.5)):
        (runs / v).mkdir(parents=True)
        (runs / v / "cpu.json").write_text(json.dumps(_doc("cpu<suite>", scale)))
        (runs / v / "manifest.json").write_text(json.dumps({"version": v, "git_sha": "a" * 40, "date": "2026-01-01"}))
    (runs / "v0.2.0" / "broken.json").write_text("{not json")
    (runs / "empty").mkdir()
    pages = R.render_site(runs, out)
    assert [p.name for p in pages] == ["index.html", "v0.1.0.html", "v0.2.0.html"]
    idx = (out / "index.html").read_text()
    assert "v0.1.0.html" in idx and "aaaaaaaaaaaa" in idx and "empty" not in idx
    page = (out / "v0.2.0.html").read_text()
    assert "cpu&lt;suite&gt;" in page and "<suite>" not in page and "matmul.128x128x128" in page and "0.5500" in page
    assert R.main(["site", "--runs-dir", str(runs), "--out", str(out)]) == 0


def test_queue_logs_every_step_survives_optional_failures_and_marks_completion(tmp_path):
    ran = []

    def ok(name):
        return lambda: ran.append(name)

    def boom():
        raise RuntimeError("no torch here")
    steps = [("first", False, ok("first")), ("optional twin", True, boom), ("last", False, ok("last"))]
    res = R.run_queue(tmp_path, [], 1, 0, "off", "0", "cpu", strict=False, steps_override=steps)
    assert ran == ["first", "last"] and res["failures"] == 0
    assert [s for _, s in res["steps"]] == ["ok", "failed: RuntimeError: no torch here", "ok"]
    log = open(res["log"]).read()
    assert "[1/3] first" in log and "FAILED (optional, continuing)" in log and "queue done: 0 failure(s)" in log
    latest = tmp_path / "queue_logs" / "latest"
    assert (latest / "done").read_text().strip() == "0" and (latest / "run.log").exists()
    res = R.run_queue(tmp_path, [], 1, 0, "off", "0", "cpu", strict=True, steps_override=steps)
    assert res["failures"] == 1


def test_queue_runs_the_cpu_suite_and_writes_the_comparative_report(tmp_path):
    res = R.run_queue(tmp_path, ["cpu"], repeats=1, warmup=0, nlp="off", seeds="0", device="cpu", strict=False)
    assert res["failures"] == 0 and [s for _, s in res["steps"]] == ["ok", "ok"]
    text = open(res["report"]).read()
    assert "Micro-benchmarks" in text and "matmul.128x128x128" in text
    assert len(list((tmp_path / "results").glob("*_cpu.json"))) == 1


def test_schema_files_accept_what_the_package_writes_and_name_what_is_wrong(tmp_path):
    from rustral_b200.bench import manifest as M
    from rustral_b200.bench import schemas
    doc = _doc("s", 1.0)
    assert schemas.check(doc, "schema_v2") == [] and schemas.check(R.combine([doc, _doc("t", 2.0)]), "schema_v2") == []
    bad = json.loads(json.dumps(doc))
    bad["schema_version"] = "1.0.0"
    bad["samples"][0]["runs_ms"] = []
    del bad["samples"][1]["dtype"]
    bad["samples"][1]["outliers"] = [0.5]
    errs = schemas.check(bad, "schema_v2")
    assert any("$.schema_version" in e for e in errs) and any("$.samples[0].runs_ms: needs at least 1" in e for e in errs)
    assert any("$.samples[1]: missing key 'dtype'" in e for e in errs) and any("$.samples[1].outliers[0]: expected integer" in e for e in errs)
    man = M.write_manifest(str(tmp_path / "m.json"), "sst2_classifier", {
        "model_type": "transformer_encoder", "seed": 1, "total_params": 10, "vocab_size": 5, "epochs": 1, "batch_size": 2,
        "learning_rate": 1e-3, "dataset_hash_fnv1a": "0123456789abcdef", "train_elapsed_sec": 0.5, "dataset": "d", "tokenizer": "t",
        "quick_mode": True, "dev_accuracy": 0.5, "dev_loss": 0.7, "samples_per_sec": 10.0},
        {"train_label_counts": [1, 1], "dev_label_counts": [1, 1], "dev_confusion_matrix": [[1, 0], [0, 1]],
         "dev_predicted_counts": [1, 1], "dev_positive_prob_hist": [0] * 10})
    assert schemas.check(man, "manifest_schema") == []
    assert any("dataset_hash_fnv1a" in e for e in schemas.check({**man, "dataset_hash_fnv1a": "xyz"}, "manifest_schema"))
    assert any("is not one of" in e for e in schemas.check({**man, "task": "other"}, "manifest_schema"))
    cur = M.curate("sst2_classifier", "dev_accuracy", "v0", [dict(man, seed=s) for s in (1, 2)])
    assert schemas.check(cur, "curated_manifest_schema") == []
    assert any("$.runs: needs at least 1" in e for e in schemas.check({**cur, "runs": []}, "curated_manifest_schema"))
    with pytest.raises(KeyError):
        schemas.load("nope")
