"""Benchmark orchestration and reporting around the schema-v2 harness documents of `rustral_b200.bench`.

    python -m rustral_b200.bench.reports run-all --suite cpu --suite torch-cpu --repeats 5 --out results/
    python -m rustral_b200.bench.reports compare --harness results/<stamp>.json --runs runs/v0.1.0 --out report.md
    python -m rustral_b200.bench.reports index --runs-dir runs [--check]
    python -m rustral_b200.bench.reports bmf combined.json bmf.json
    python -m rustral_b200.bench.reports emnlp --harness combined.json --runs runs/v0.1.0 --out emnlp_report.md
    python -m rustral_b200.bench.reports regress --baseline old.json --current new.json --fail-on-regression
    python -m rustral_b200.bench.reports site --runs-dir runs --out site/
    python -m rustral_b200.bench.reports queue --out benchmarks [--nlp benchmark|paper|off] [--strict]

What each sub-command does, and the script of the reference whose job it takes over:

* run-all   runs one or more suites (this framework on CPU / on the B200, plain PyTorch on CPU / CUDA as the
            comparison arm) over the shared workload list, merges the per-suite documents into one combined document
            and writes it with a Markdown summary (scripts/bench/run_all.py:1-314; the JAX / TensorFlow /
            ONNX-Runtime suites of the reference are not offered: those packages are not part of this installation);
* compare   a comparative Markdown report: per-workload table across suites with the speed-up against a chosen
            baseline suite, and the NLP task aggregates (mean +- std over seeds) of this framework next to the PyTorch
            twins (scripts/bench/comparative_report.py);
* index     regenerates `INDEX.md` from every `<runs-dir>/<version>/manifest.json`, or with --check fails when the
            file on disk is stale (scripts/bench/regen_index.py);
* bmf       converts a combined document into Bencher Metric Format: `<suite>/<backend>/<device>/<name>` ->
            latency in ns with lower / upper values (scripts/bench/to_bencher_bmf.py);
* emnlp     the paper-style experiment report: environment, micro-benchmark tables per suite, NLP tables
            (scripts/bench/build_emnlp_report.py);
* regress   a regression gate between two harness documents: workloads are matched by (suite, name, params), the ratio
            of means is reported, and with --fail-on-regression the exit status is 1 when a workload is slower than
            --max-slowdown times the baseline AND the two 95 % confidence intervals do not overlap (so noise alone does
            not fail a build); --require-matching fails on workloads that disappeared
            (scripts/bench/compare_harness.py);
* queue     the whole measurement campaign as one sequential job list with a log: micro-benchmark suites of this
            framework, the plain-PyTorch suites, the multi-seed NLP evaluation, its PyTorch twins, and the comparative
            report at the end.  Every step is time-stamped in `<out>/queue_logs/<stamp>/run.log` (`latest` points at the
            newest), a failing optional step is recorded and skipped over (with --strict it fails the run), and a
            `done` file marks completion (scripts/bench/queue_all_benchmarks.sh, scripts/run_paper_experiments.sh);
* site      a static HTML dashboard: `index.html` listing every snapshot under --runs-dir with its manifest, and one
            page per snapshot with a sortable table per suite; no scripts are fetched and nothing is loaded at view
            time (scripts/bench/render_site.py).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import time
from pathlib import Path

from . import SCHEMA_VERSION, Sample, ci95_mean_ms, machine_info, samples_to_json, time_runs, validate_schema

SUITES = ("cpu", "b200", "torch-cpu", "torch-cuda")


# ------------------------------------------------------------------------------------------------- plain-PyTorch suite
def _torch_workloads(device: str, heavy: bool) -> list:
    """The comparison arm: the workloads of `workloads.build_workloads` (same names and shapes) written with stock
    torch modules only."""
    import torch
    import torch.nn.functional as F
    dev = torch.device(device)
    g = torch.Generator().manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g).to(dev)
    out = []
    for n in (128, 256, 512):
        a, b = rnd(n, n), rnd(n, n)
        out.append((f"matmul.{n}x{n}x{n}", {"m": n, "k": n, "n": n}, lambda a=a, b=b: a @ b, 0))
    for r, c in ((32, 64), (32, 256), (64, 1024)):
        x = rnd(r, c)
        out.append((f"softmax_dim.{r}x{c}", {"rows": r, "cols": c}, lambda x=x: torch.softmax(x, -1), 0))
    for b_, i, o in ((32, 256, 1024), (32, 1024, 256)):
        lin = torch.nn.Linear(i, o).to(dev)
        x = rnd(b_, i)
        out.append((f"fused_linear_bias_gelu.{b_}x{i}->{o}", {"batch": b_, "in": i, "out": o},
                    lambda lin=lin, x=x: F.gelu(lin(x), approximate="tanh"), sum(p.numel() for p in lin.parameters())))
    for name, d, h, s_ in (("attention.small", 64, 4, 32), ("attention.medium", 256, 8, 128)):
        q, k, v = (rnd(1, h, s_, d // h) for _ in range(3))
        out.append((name, {"d_model": d, "heads": h, "seq": s_, "head_dim": d // h},
                    lambda q=q, k=k, v=v: F.scaled_dot_product_attention(q, k, v), 0))
    for name, c, hw, o in (("conv2d.small", 1, 28, 8), ("conv2d.medium", 3, 64, 16), ("conv2d.large", 3, 224, 32)):
        conv = torch.nn.Conv2d(c, o, 3).to(dev)
        x = rnd(4, c, hw, hw)
        out.append((name, {"channels": c, "hw": hw, "out": o}, lambda conv=conv, x=x: conv(x), sum(p.numel() for p in conv.parameters())))
    for name, hsz, steps in (("lstm_forward.small", 128, 10), ("lstm_forward.medium", 256, 50), ("lstm_forward.large", 512, 100)):
        lstm = torch.nn.LSTM(hsz, hsz).to(dev)
        xs = rnd(steps, 1, hsz)
        out.append((name, {"hidden": hsz, "steps": steps}, lambda lstm=lstm, xs=xs: lstm(xs), sum(p.numel() for p in lstm.parameters())))
    mlp = torch.nn.Sequential(torch.nn.Linear(128, 256), torch.nn.ReLU(), torch.nn.Linear(256, 64)).to(dev)
    opt = torch.optim.Adam(mlp.parameters(), lr=1e-3)
    xb, yb = rnd(32, 128), rnd(32, 64)

    def mlp_step():
        opt.zero_grad(set_to_none=True)
        loss = ((mlp(xb) - yb) ** 2).mean()
        loss.backward()
        opt.step()
    out.append(("mlp_train_step", {"batch": 32, "dims": [128, 256, 64]}, mlp_step, sum(p.numel() for p in mlp.parameters())))
    n_opt = 100_000_000 if heavy else 10_000_000
    slabs = [torch.nn.Parameter(torch.zeros(n_opt // 8, device=dev)) for _ in range(8)]
    for p_ in slabs:
        p_.grad = torch.ones_like(p_)
    sgd, adam = torch.optim.SGD(slabs, lr=0.01), torch.optim.Adam(slabs, lr=1e-3)
    out.append(("optimizer_step.sgd", {"params": n_opt}, lambda: sgd.step(), n_opt))
    out.append(("optimizer_step.adam", {"params": n_opt}, lambda: adam.step(), n_opt))
    layer = torch.nn.TransformerEncoderLayer(128, 4, 512, dropout=0.0, activation="gelu", batch_first=True, norm_first=True)
    enc = torch.nn.TransformerEncoder(layer, 2, enable_nested_tensor=False).to(dev)
    emb = torch.nn.Embedding(1024, 128).to(dev)
    ids = torch.randint(0, 1024, (1, 128), generator=g).to(dev)
    out.append(("transformer_encoder.forward", {"layers": 2, "d_model": 128, "heads": 4, "ffn": 512, "seq": 128, "vocab": 1024},
                lambda: enc(emb(ids)), sum(p.numel() for p in enc.parameters()) + emb.weight.numel()))
    return out


def run_torch_suite(device: str, repeats: int, warmup: int, heavy: bool = False) -> dict:
    import torch
    samples = []
    for name, params, fn, nparams in _torch_workloads(device, heavy):
        if name == "mlp_train_step" or name.startswith("optimizer_step"):
            runs = time_runs(fn, warmup, repeats, cuda=(device != "cpu"))
        else:
            with torch.no_grad():
                runs = time_runs(fn, warmup, repeats, cuda=(device != "cpu"))
        samples.append(Sample(name, "pytorch", device if device == "cpu" else "cuda", "f32", nparams, params, runs))
    return json.loads(samples_to_json(samples, suite="torch-" + ("cpu" if device == "cpu" else "cuda")))


def run_suite(suite: str, repeats: int, warmup: int, heavy: bool = False) -> dict | None:
    """One suite's schema-v2 document, or None when the suite cannot run here (no GPU for the CUDA suites)."""
    import torch
    if suite in ("b200", "torch-cuda") and not torch.cuda.is_available():
        return None
    if suite in ("cpu", "b200"):
        from . import workloads
        doc = json.loads(workloads.run("cpu" if suite == "cpu" else "cuda", repeats, warmup, heavy))
        doc["suite"] = "rustral-b200-" + ("cpu" if suite == "cpu" else "b200")
        return doc
    if suite in ("torch-cpu", "torch-cuda"):
        return run_torch_suite("cpu" if suite == "torch-cpu" else "cuda", repeats, warmup, heavy)
    raise ValueError(f"unknown suite {suite!r}; choose from {SUITES}")


def combine(docs: list) -> dict:
    """Merges suite documents into one combined document: the samples carry their suite name."""
    samples = []
    for d in docs:
        for s in d["samples"]:
            samples.append(dict(s, suite=d["suite"]))
    return {"schema_version": SCHEMA_VERSION, "suite": "combined", "suites": [d["suite"] for d in docs],
            "machine": docs[0]["machine"] if docs else machine_info(), "samples": samples}


def _key(s: dict) -> str:
    return s["name"]


def summary_markdown(doc: dict, baseline_suite: str | None = None) -> str:
    """Per-workload table: one column per suite (mean ms +- 95 % CI), optional speed-up against `baseline_suite`."""
    suites = list(dict.fromkeys(s.get("suite", doc.get("suite", "?")) for s in doc["samples"]))
    rows: dict = {}
    for s in doc["samples"]:
        rows.setdefault(_key(s), {})[s.get("suite", doc.get("suite", "?"))] = s
    head = ["workload"] + suites + ([f"speed-up vs {baseline_suite}"] if baseline_suite else [])
    lines = ["| " + " | ".join(head) + " |", "|" + "---|" * len(head)]
    for k, by in rows.items():
        cells = [k]
        for su in suites:
            s = by.get(su)
            if s is None:
                cells.append("-")
                continue
            ci = s.get("ci95_ms")
            cells.append(f"{s['mean_ms']:.4f}" + (f" +- {ci:.4f}" if ci else ""))
        if baseline_suite:
            base = by.get(baseline_suite)
            best = [by[su]["mean_ms"] for su in suites if su != baseline_suite and su in by]
            cells.append(f"{base['mean_ms'] / min(best):.2f}x" if base and best and min(best) > 0 else "-")
        lines.append("| " + " | ".join(cells) + " |")
    return "\n".join(lines) + "\n"


def cmd_run_all(a) -> int:
    docs = []
    for su in a.suite or ["cpu", "torch-cpu"]:
        d = run_suite(su, a.repeats, a.warmup, a.heavy)
        if d is None:
            print(f"suite {su}: skipped (needs a CUDA device)", file=sys.stderr)
            continue
        errs = validate_schema(d)
        if errs:
            raise SystemExit(f"suite {su} produced an invalid document: {errs}")
        docs.append(d)
    if not docs:
        raise SystemExit("no suite could run")
    doc = combine(docs)
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    stamp = time.strftime("%Y%m%d_%H%M%S")
    (out / f"{stamp}.json").write_text(json.dumps(doc, indent=1))
    (out / "summary.md").write_text(f"# Benchmark summary ({stamp})\n\n" + summary_markdown(doc, a.baseline))
    print(out / f"{stamp}.json")
    return 0


# ------------------------------------------------------------------------------------------------- comparative report
def _mean_std(xs: list) -> tuple:
    if not xs:
        return float("nan"), float("nan")
    return (float(xs[0]), 0.0) if len(xs) == 1 else (statistics.mean(xs), statistics.stdev(xs))


def _pm(m: float, s: float, nd: int = 4) -> str:
    if m != m:
        return "n/a"
    return f"{m:.{nd}f}" if not s or s != s else f"{m:.{nd}f} +- {s:.{nd}f}"


def nlp_section(title: str, ours: Path, twin: Path, metric: str) -> str:
    """Mean +- std over seeds of `metric` and of the training throughput for this framework and its PyTorch twin
    (curated documents written by `bench.manifest.curate`)."""
    lines = [f"## {title}", ""]
    for label, path in (("this framework", ours), ("PyTorch twin", twin)):
        if path is None or not path.exists():
            lines.append(f"*{label}: no curated file at `{path}`*")
            continue
        doc = json.loads(path.read_text())
        # a curated run is {"seed", "manifest": {...}}: the metric is the document's own `metric` key (dev_accuracy,
        # dev_perplexity) inside the manifest, the rate is samples or tokens per second; flat runs are accepted as well
        runs = [r.get("manifest", r) if isinstance(r, dict) else {} for r in doc.get("runs", [])]
        keys = [k for k in (doc.get("metric"), metric, "dev_" + metric) if k]
        vals = [next(float(r[k]) for k in keys if isinstance(r.get(k), (int, float))) for r in runs
                if any(isinstance(r.get(k), (int, float)) for k in keys)]
        rate_keys = ("throughput", "tokens_per_sec", "samples_per_sec")
        thr = [next(float(r[k]) for k in rate_keys if isinstance(r.get(k), (int, float))) for r in runs
               if any(isinstance(r.get(k), (int, float)) for k in rate_keys)]
        lines.append(f"* {label}: {metric} {_pm(*_mean_std(vals))} over {len(vals)} seed(s); "
                     f"throughput {_pm(*_mean_std(thr), nd=1)} per second")
    return "\n".join(lines) + "\n"


def cmd_compare(a) -> int:
    parts = [f"# Comparative report ({time.strftime('%Y-%m-%d')})", ""]
    if a.harness:
        docs = [json.loads(Path(p).read_text()) for p in a.harness]
        merged = docs[0] if len(docs) == 1 and docs[0].get("suite") == "combined" else combine(
            [d for d in docs if d.get("suite") != "combined"] or docs)
        m = merged.get("machine", {})
        parts += ["## Micro-benchmarks", "", f"Machine: {m.get('os', '?')} / {m.get('cpu', '?')} / {m.get('gpu', 'no GPU')}", "",
                  summary_markdown(merged, a.baseline)]
    if a.runs:
        base = Path(a.runs)
        parts.append(nlp_section("SST-2 classifier (dev accuracy)", base / "nlp" / "sst2.json", base / "nlp" / "sst2_pytorch.json", "accuracy"))
        parts.append(nlp_section("WikiText-2 word LM (dev perplexity)", base / "nlp" / "wikitext2.json",
                                 base / "nlp" / "wikitext2_pytorch.json", "perplexity"))
    text = "\n".join(parts)
    if a.out:
        Path(a.out).parent.mkdir(parents=True, exist_ok=True)
        Path(a.out).write_text(text)
    else:
        print(text)
    return 0


def cmd_emnlp(a) -> int:
    """The experiment report: environment block, one micro-benchmark table per suite, the NLP aggregates."""
    parts = ["# Experiments report", "", "## Environment", ""]
    docs = [json.loads(Path(p).read_text()) for p in (a.harness or [])]
    m = (docs[0].get("machine") if docs else None) or machine_info()
    parts += [f"* {k}: {v}" for k, v in m.items()] + [""]
    for d in docs:
        for su in (d.get("suites") or [d.get("suite")]):
            rows = [s for s in d["samples"] if s.get("suite", d.get("suite")) == su]
            if not rows:
                continue
            parts += [f"## Micro-benchmarks: {su}", "", "| workload | mean ms | 95 % CI | min ms | runs |", "|---|---|---|---|---|"]
            for s in rows:
                ci = s.get("ci95_ms")
                parts.append(f"| {_key(s)} | {s['mean_ms']:.4f} | {ci:.4f} | {s.get('min_ms', float('nan')):.4f} | {len(s['runs_ms'])} |"
                             if ci else f"| {_key(s)} | {s['mean_ms']:.4f} | - | {s.get('min_ms', float('nan')):.4f} | {len(s['runs_ms'])} |")
            parts.append("")
    if a.runs:
        base = Path(a.runs)
        parts.append(nlp_section("SST-2", base / "nlp" / "sst2.json", base / "nlp" / "sst2_pytorch.json", "accuracy"))
        parts.append(nlp_section("WikiText-2", base / "nlp" / "wikitext2.json", base / "nlp" / "wikitext2_pytorch.json", "perplexity"))
    Path(a.out).parent.mkdir(parents=True, exist_ok=True)
    Path(a.out).write_text("\n".join(parts))
    return 0


# ------------------------------------------------------------------------------------------------- release index
INDEX_BOUNDARY = "## Index"
_REQUIRED = ("version", "git_sha", "date")


def index_table(runs_dir: Path) -> str:
    rows = []
    for mf in sorted(runs_dir.glob("*/manifest.json")):
        doc = json.loads(mf.read_text())
        missing = [k for k in _REQUIRED if k not in doc]
        if missing:
            raise ValueError(f"{mf}: missing keys {missing}")
        suites = sorted(p.stem for p in mf.parent.glob("*.json") if p.name != "manifest.json")
        rows.append((doc["version"], doc["date"], doc["git_sha"][:12], doc.get("machine", "?"), ", ".join(suites) or "-"))
    lines = ["| version | date | git sha | machine | suites |", "|---|---|---|---|---|"]
    lines += ["| " + " | ".join(r) + " |" for r in rows]
    return "\n".join(lines) + "\n"


def cmd_index(a) -> int:
    runs = Path(a.runs_dir)
    index = runs / "INDEX.md"
    head = index.read_text().split(INDEX_BOUNDARY)[0] if index.exists() else "# Benchmark snapshots\n\n"
    want = head + INDEX_BOUNDARY + "\n\n" + index_table(runs)
    if a.check:
        if not index.exists() or index.read_text() != want:
            print(f"{index} is stale: run `python -m rustral_b200.bench.reports index --runs-dir {runs}`", file=sys.stderr)
            return 1
        return 0
    index.write_text(want)
    return 0


# ------------------------------------------------------------------------------------------------- Bencher Metric Format
def to_bmf(doc: dict) -> dict:
    out = {}
    for s in doc["samples"]:
        name = "/".join([s.get("suite", doc.get("suite", "?")), s["backend"], s["device"], _key(s)])
        runs = s["runs_ms"]
        out[name] = {"latency": {"value": statistics.mean(runs) * 1e6, "lower_value": min(runs) * 1e6, "upper_value": max(runs) * 1e6}}
    return out


def cmd_bmf(a) -> int:
    src = sys.stdin.read() if a.input == "-" else Path(a.input).read_text()
    Path(a.output).write_text(json.dumps(to_bmf(json.loads(src)), indent=1))
    return 0


# ------------------------------------------------------------------------------------------------- regression gate
def _sample_index(doc: dict) -> dict:
    """(suite, name, sorted params) -> sample, for per-suite and combined documents alike."""
    out = {}
    for s in doc.get("samples") or []:
        params = s.get("params") if isinstance(s.get("params"), dict) else {}
        out[(str(s.get("suite", doc.get("suite", "?"))), str(s.get("name", "")), tuple(sorted((str(k), str(v)) for k, v in params.items())))] = s
    return out


def _interval(s: dict) -> tuple:
    ci = s.get("ci95_ms")
    if ci is None and len(s.get("runs_ms") or []) >= 2:
        ci = ci95_mean_ms(s["runs_ms"])
    m = float(s["mean_ms"])
    return (m - ci, m + ci) if ci else (m, m)


def regress(base: dict, cur: dict, max_slowdown: float = 1.15) -> dict:
    """Rows of matched workloads with their ratio; a row is a regression when it is slower than `max_slowdown` times the
    baseline and the confidence intervals of the two means are disjoint."""
    bi, ci = _sample_index(base), _sample_index(cur)
    rows, skipped = [], []
    for k in sorted(bi):
        if k not in ci:
            continue
        bm, cm = bi[k].get("mean_ms"), ci[k].get("mean_ms")
        if not isinstance(bm, (int, float)) or not isinstance(cm, (int, float)) or bm <= 0 or not math.isfinite(cm):
            skipped.append(k)
            continue
        ratio = cm / bm
        (_, b_hi), (c_lo, _) = _interval(bi[k]), _interval(ci[k])
        rows.append({"suite": k[0], "name": k[1], "params": dict(k[2]), "baseline_ms": bm, "current_ms": cm, "ratio": ratio,
                     "regression": ratio > max_slowdown and c_lo > b_hi})
    return {"rows": rows, "skipped": skipped, "missing": [k for k in sorted(bi) if k not in ci],
            "extra": [k for k in sorted(ci) if k not in bi]}


def cmd_regress(a) -> int:
    res = regress(json.loads(Path(a.baseline).read_text()), json.loads(Path(a.current).read_text()), a.max_slowdown)
    bad = [r for r in res["rows"] if r["regression"]]
    print(f"compared {len(res['rows'])} workloads ({len(res['skipped'])} without a usable mean); {len(bad)} regression(s) "
          f"beyond {a.max_slowdown:.2f}x")
    for r in res["rows"]:
        label = r["name"] + ("." + ".".join(f"{k}={v}" for k, v in r["params"].items()) if r["params"] else "")
        print(f"  {r['suite']:<12} {label:<48} {r['baseline_ms']:>10.4f} -> {r['current_ms']:>10.4f} ms   x{r['ratio']:.3f}"
              + ("   REGRESSION" if r["regression"] else ""))
    for title, keys in (("missing in current", res["missing"]), ("new in current", res["extra"])):
        if keys:
            print(f"{title}: " + ", ".join(f"{k[0]}/{k[1]}" for k in keys[:40]) + (" ..." if len(keys) > 40 else ""))
    if a.require_matching and res["missing"]:
        print("FAIL: workloads of the baseline are missing in the current document", file=sys.stderr)
        return 1
    if a.fail_on_regression and bad:
        print(f"FAIL: {len(bad)} workload(s) regressed", file=sys.stderr)
        return 1
    return 0


# ------------------------------------------------------------------------------------------------- static dashboard
_PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>{title}</title><style>
body{{font:14px/1.45 system-ui,sans-serif;margin:2rem auto;max-width:72rem;padding:0 1rem;color:#1b1f24}}
table{{border-collapse:collapse;margin:.5rem 0 1.5rem}}th,td{{border:1px solid #d0d7de;padding:.25rem .6rem;text-align:right}}
th{{background:#f6f8fa;cursor:pointer}}td:first-child,th:first-child{{text-align:left}}code{{background:#f6f8fa;padding:0 .25rem}}
</style></head><body><h1>{title}</h1>{body}<script>
document.querySelectorAll("th").forEach(function(th){{th.onclick=function(){{var t=th.closest("table"),i=th.cellIndex,
r=[].slice.call(t.tBodies[0].rows),d=th.dataset.d=th.dataset.d=="1"?"-1":"1";r.sort(function(a,b){{var x=a.cells[i].textContent,
y=b.cells[i].textContent,n=parseFloat(x)-parseFloat(y);return d*(isNaN(n)?x.localeCompare(y):n)}});r.forEach(function(e){{t.tBodies[0].appendChild(e)}})}}}});
</script></body></html>"""


def _suite_tables(docs: list) -> str:
    import html
    parts = []
    for d in docs:
        for su in (d.get("suites") or [d.get("suite", "?")]):
            rows = [s for s in d.get("samples") or [] if s.get("suite", d.get("suite")) == su]
            if not rows:
                continue
            parts.append(f"<h2>{html.escape(str(su))}</h2><table><thead><tr><th>workload</th><th>backend</th><th>device</th>"
                         "<th>mean ms</th><th>95 % CI</th><th>min ms</th><th>runs</th></tr></thead><tbody>")
            for s in rows:
                ci = s.get("ci95_ms")
                parts.append("<tr><td>{}</td><td>{}</td><td>{}</td><td>{:.4f}</td><td>{}</td><td>{:.4f}</td><td>{}</td></tr>".format(
                    html.escape(_key(s)), html.escape(str(s.get("backend", "?"))), html.escape(str(s.get("device", "?"))),
                    float(s["mean_ms"]), f"{ci:.4f}" if ci else "-", float(s.get("min_ms", min(s.get("runs_ms") or [float("nan")]))),
                    len(s.get("runs_ms") or [])))
            parts.append("</tbody></table>")
    return "".join(parts)


def render_site(runs_dir: Path, out: Path) -> list:
    """Writes index.html plus one page per `<runs-dir>/<version>/` holding harness documents; returns the written paths.
    An empty or absent runs directory still yields a valid landing page."""
    import html
    out.mkdir(parents=True, exist_ok=True)
    written, items = [], []
    versions = sorted(p for p in runs_dir.iterdir() if p.is_dir()) if runs_dir.is_dir() else []
    for vdir in versions:
        docs, manifest = [], {}
        for f in sorted(vdir.glob("*.json")):
            try:
                doc = json.loads(f.read_text())
            except json.JSONDecodeError:
                continue
            if f.name == "manifest.json":
                manifest = doc
            elif isinstance(doc, dict) and isinstance(doc.get("samples"), list):
                docs.append(doc)
        if not docs and not manifest:
            continue
        meta = "".join(f"<li>{html.escape(str(k))}: <code>{html.escape(str(v))}</code></li>" for k, v in manifest.items()
                       if not isinstance(v, (dict, list)))
        body = (f"<p><a href='index.html'>all snapshots</a></p><ul>{meta}</ul>" + (_suite_tables(docs) or "<p>no harness documents</p>"))
        page = out / f"{vdir.name}.html"
        page.write_text(_PAGE.format(title=html.escape(f"Benchmarks {vdir.name}"), body=body))
        written.append(page)
        n = sum(len(d["samples"]) for d in docs)
        items.append(f"<tr><td><a href='{html.escape(vdir.name)}.html'>{html.escape(vdir.name)}</a></td><td>{html.escape(str(manifest.get('date', '-')))}</td>"
                     f"<td>{html.escape(str(manifest.get('git_sha', '-'))[:12])}</td><td>{len(docs)}</td><td>{n}</td></tr>")
    body = ("<table><thead><tr><th>snapshot</th><th>date</th><th>git sha</th><th>suites</th><th>workloads</th></tr></thead><tbody>"
            + "".join(items) + "</tbody></table>") if items else "<p>no snapshots yet</p>"
    index = out / "index.html"
    index.write_text(_PAGE.format(title="Benchmark snapshots", body=body))
    return [index] + written


def cmd_site(a) -> int:
    for p in render_site(Path(a.runs_dir), Path(a.out)):
        print(p)
    return 0


# ------------------------------------------------------------------------------------------------- campaign queue
def run_queue(out: Path, suites: list, repeats: int, warmup: int, nlp: str, seeds: str, device: str, strict: bool,
              torch_twins: bool = True, steps_override: list | None = None) -> dict:
    """Runs the job list in order; returns {"failures": n, "steps": [(name, "ok" | "failed: ..." | "skipped")], "report": path}.
    `steps_override` replaces the job list with [(name, optional, callable)] (used by tests)."""
    stamp = time.strftime("%Y%m%d_%H%M%S")
    logdir = out / "queue_logs" / stamp
    logdir.mkdir(parents=True, exist_ok=True)
    latest = out / "queue_logs" / "latest"
    try:
        if latest.is_symlink() or latest.exists():
            latest.unlink()
        latest.symlink_to(stamp)
    except OSError:
        pass
    log_path = logdir / "run.log"
    results, harness_docs, runs_dir = [], [], out / "runs" / stamp
    report = out / "reports" / f"comparative_queue_{stamp}.md"

    def log(msg: str) -> None:
        with open(log_path, "a") as f:
            f.write(f"[{time.strftime('%Y-%m-%dT%H:%M:%S')}] {msg}\n")

    def suites_step(names):
        def go():
            docs = [d for d in (run_suite(su, repeats, warmup) for su in names) if d is not None]
            if not docs:
                raise RuntimeError("no suite of this step can run on this machine")
            doc = combine(docs)
            path = out / "results" / f"{stamp}_{'_'.join(names)}.json"
            path.parent.mkdir(parents=True, exist_ok=True)
            path.write_text(json.dumps(doc, indent=1))
            harness_docs.append(str(path))
        return go

    def nlp_step():
        from . import nlp_eval
        rc = nlp_eval.main([f"--{nlp}", "--seeds", seeds, "--device", device, "--out", str(runs_dir / "nlp"), "--clean"])
        if rc:
            raise RuntimeError(f"nlp_eval exit status {rc}")

    def twin_step(task):
        def go():
            from . import torch_baselines
            argv = ["--task", task, "--seeds", seeds, "--device", device, "--out", str(runs_dir / "nlp")]
            vocabs = sorted((runs_dir / "nlp" / "raw" / "sst2").glob("seed*/vocab.txt"))     # written by the first seed's run
            if task == "sst2" and vocabs:
                argv += ["--vocab", str(vocabs[0])]
            if nlp == "benchmark":
                argv.append("--quick")
            rc = torch_baselines.main(argv)
            if rc:
                raise RuntimeError(f"torch_baselines exit status {rc}")
        return go

    def report_step():
        ns = argparse.Namespace(harness=harness_docs or None, runs=str(runs_dir) if (runs_dir / "nlp").is_dir() else None,
                                baseline=None, out=str(report))
        cmd_compare(ns)

    ours = [su for su in suites if not su.startswith("torch")]
    theirs = [su for su in suites if su.startswith("torch")]
    steps = steps_override
    if steps is None:
        steps = []
        if ours:
            steps.append((f"micro-benchmarks: {', '.join(ours)}", False, suites_step(ours)))
        if theirs:
            steps.append((f"micro-benchmarks: {', '.join(theirs)}", True, suites_step(theirs)))
        if nlp != "off":
            steps.append((f"NLP evaluation ({nlp}, seeds {seeds})", False, nlp_step))
            if torch_twins:
                steps += [("PyTorch twin: sst2", True, twin_step("sst2")), ("PyTorch twin: wikitext2", True, twin_step("wikitext2"))]
        steps.append(("comparative report", False, report_step))
    failures = 0
    log(f"queue start: {len(steps)} step(s), out={out}")
    for i, (name, optional, fn) in enumerate(steps, 1):
        log(f"=== [{i}/{len(steps)}] {name} ===")
        t0 = time.perf_counter()
        try:
            fn()
            results.append((name, "ok"))
            log(f"[{i}] ok in {time.perf_counter() - t0:.1f} s")
        except (Exception, SystemExit) as e:      # noqa: BLE001 - a failed step must not stop the queue
            results.append((name, f"failed: {type(e).__name__}: {e}"))
            if optional and not strict:
                log(f"[{i}] FAILED (optional, continuing): {type(e).__name__}: {e}")
            else:
                failures += 1
                log(f"[{i}] FAILED: {type(e).__name__}: {e}")
    log(f"queue done: {failures} failure(s)")
    (logdir / "done").write_text(f"{failures}\n")
    return {"failures": failures, "steps": results, "report": str(report), "log": str(log_path)}


def cmd_queue(a) -> int:
    res = run_queue(Path(a.out), a.suite or ["cpu", "b200", "torch-cpu", "torch-cuda"], a.repeats, a.warmup, a.nlp, a.seeds, a.device,
                    a.strict, not a.no_torch_twins)
    for name, status in res["steps"]:
        print(f"{status.split(':')[0]:<7} {name}")
    print(f"log: {res['log']}\nreport: {res['report']}")
    return 1 if res["failures"] else 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="rustral_b200.bench.reports")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("run-all")
    p.add_argument("--suite", action="append", choices=SUITES)
    p.add_argument("--repeats", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--heavy", action="store_true")
    p.add_argument("--baseline", default=None, help="suite the speed-up column is computed against")
    p.add_argument("--out", default="benchmarks/results")
    p.set_defaults(fn=cmd_run_all)
    p = sub.add_parser("compare")
    p.add_argument("--harness", action="append")
    p.add_argument("--runs", default=None, help="a snapshot directory with nlp/<task>.json and nlp/<task>_pytorch.json")
    p.add_argument("--baseline", default=None)
    p.add_argument("--out", default=None)
    p.set_defaults(fn=cmd_compare)
    p = sub.add_parser("emnlp")
    p.add_argument("--harness", action="append")
    p.add_argument("--runs", default=None)
    p.add_argument("--out", required=True)
    p.set_defaults(fn=cmd_emnlp)
    p = sub.add_parser("index")
    p.add_argument("--runs-dir", required=True)
    p.add_argument("--check", action="store_true")
    p.set_defaults(fn=cmd_index)
    p = sub.add_parser("bmf")
    p.add_argument("input")
    p.add_argument("output")
    p.set_defaults(fn=cmd_bmf)
    p = sub.add_parser("regress")
    p.add_argument("--baseline", required=True)
    p.add_argument("--current", required=True)
    p.add_argument("--max-slowdown", type=float, default=1.15, help="allowed current mean / baseline mean")
    p.add_argument("--fail-on-regression", action="store_true")
    p.add_argument("--require-matching", action="store_true", help="fail when a baseline workload is absent from the current document")
    p.set_defaults(fn=cmd_regress)
    p = sub.add_parser("queue")
    p.add_argument("--out", default="benchmarks")
    p.add_argument("--suite", action="append", choices=SUITES, help="default: every suite (those that need a GPU are skipped without one)")
    p.add_argument("--repeats", type=int, default=5)
    p.add_argument("--warmup", type=int, default=1)
    p.add_argument("--nlp", choices=["benchmark", "paper", "off"], default="benchmark")
    p.add_argument("--seeds", default="0,1,2")
    p.add_argument("--device", default="cpu")
    p.add_argument("--no-torch-twins", action="store_true")
    p.add_argument("--strict", action="store_true", help="optional steps that fail count as failures")
    p.set_defaults(fn=cmd_queue)
    p = sub.add_parser("site")
    p.add_argument("--runs-dir", required=True)
    p.add_argument("--out", required=True)
    p.set_defaults(fn=cmd_site)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
