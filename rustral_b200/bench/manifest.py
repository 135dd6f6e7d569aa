"""Run manifests: the JSON record an example or benchmark run leaves next to its outputs, and the curated multi-seed
files built from them (benchmarks/manifest_schema.json, scripts/bench/validate_manifest.py,
crates/runtime/examples/sst2_classifier.rs:722-757).

A run manifest is a flat object: task, model_type, git_sha, seed, hyper-parameters, dataset sizes and FNV-1a hash,
the task's metric(s), throughput and a `diagnostics` object.  A curated manifest wraps several runs:
{schema_version, created_at, version, task, metric, aggregate{mean, std, n}, runs[{seed, manifest}]}.
"""
from __future__ import annotations

import datetime
import json
import math
import os
import subprocess

MANIFEST_SCHEMA_VERSION = "1.0.0"

RUN_REQUIRED = ("task", "model_type", "git_sha", "seed", "total_params", "vocab_size", "epochs", "batch_size",
                "learning_rate", "dataset_hash_fnv1a", "train_elapsed_sec", "dataset", "tokenizer", "quick_mode")
TASK_METRICS = {"sst2_classifier": ("dev_accuracy", "dev_loss"),
                "wikitext2_word_lm": ("dev_perplexity", "dev_loss_nats"),
                "emnlp_char_lm": ("dev_perplexity", "dev_loss_nats")}
SST2_DIAGNOSTICS = ("train_label_counts", "dev_label_counts", "dev_confusion_matrix", "dev_predicted_counts",
                    "dev_positive_prob_hist")
CURATED_REQUIRED = ("schema_version", "created_at", "version", "task", "metric", "aggregate", "runs")


def detect_git_sha(cwd: str | None = None) -> str:
    """HEAD of the repository that holds `cwd` (the package's own checkout by default); "unknown" outside git."""
    cwd = cwd or os.path.dirname(os.path.abspath(__file__))
    try:
        out = subprocess.run(["git", "rev-parse", "HEAD"], cwd=cwd, capture_output=True, text=True, timeout=5)
        sha = out.stdout.strip()
        return sha if out.returncode == 0 and sha else "unknown"
    except (OSError, subprocess.SubprocessError):
        return "unknown"


def _json_safe(v):
    if isinstance(v, float) and not math.isfinite(v):
        return None
    if isinstance(v, dict):
        return {str(k): _json_safe(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_json_safe(x) for x in v]
    if hasattr(v, "item") and not isinstance(v, (str, bytes)):
        return _json_safe(v.item())
    return v


def write_manifest(path: str, task: str, fields: dict, diagnostics: dict | None = None) -> dict:
    """Writes `<path>` (a file, or a directory that receives manifest.json) and returns the document.  `git_sha` is
    filled in when the caller did not give one; non-finite floats become null so the file stays strict JSON."""
    doc = {"task": task}
    doc.update(fields)
    doc.setdefault("git_sha", detect_git_sha())
    doc["diagnostics"] = diagnostics or {}
    doc = _json_safe(doc)
    if os.path.isdir(path) or path.endswith(os.sep):
        os.makedirs(path, exist_ok=True)
        path = os.path.join(path, "manifest.json")
    else:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = path + ".tmp"
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(doc, f, indent=2, sort_keys=False)
        f.write("\n")
    os.replace(tmp, path)
    return doc


def validate_manifest(doc: dict, where: str = "<manifest>") -> list:
    """Problems of one RUN manifest as a list of strings (empty = valid)."""
    errs = []
    if not isinstance(doc, dict):
        return [f"{where}: must be an object"]
    missing = [k for k in RUN_REQUIRED if k not in doc]
    if missing:
        errs.append(f"{where}: missing keys: {missing}")
    task = doc.get("task")
    for k in TASK_METRICS.get(task, ()):
        if k not in doc:
            errs.append(f"{where}: task {task} requires {k}")
        elif doc[k] is not None and not isinstance(doc[k], (int, float)):
            errs.append(f"{where}: {k} must be a number")
    if task == "sst2_classifier" and doc.get("framework") != "pytorch":
        diag = doc.get("diagnostics")
        if not isinstance(diag, dict):
            errs.append(f"{where}: diagnostics is required for sst2_classifier")
        else:
            miss = [k for k in SST2_DIAGNOSTICS if k not in diag]
            if miss:
                errs.append(f"{where}: diagnostics missing keys: {miss}")
    for k in ("seed", "epochs", "batch_size", "total_params", "vocab_size"):
        if k in doc and not (isinstance(doc[k], int) and not isinstance(doc[k], bool) and doc[k] >= 0):
            errs.append(f"{where}: {k} must be a non-negative integer")
    return errs


def curate(task: str, metric: str, version: str, manifests: list) -> dict:
    """Wraps the run manifests of several seeds into one curated document with mean / sample-std of `metric`."""
    vals = [float(m[metric]) for m in manifests if m.get(metric) is not None]
    n = len(vals)
    mean = sum(vals) / n if n else float("nan")
    std = math.sqrt(sum((v - mean) ** 2 for v in vals) / (n - 1)) if n > 1 else 0.0
    return _json_safe({
        "schema_version": MANIFEST_SCHEMA_VERSION,
        "created_at": datetime.datetime.now(datetime.timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ"),
        "version": version, "task": task, "metric": metric,
        "aggregate": {"mean": mean, "std": std, "n": n},
        "runs": [{"seed": m.get("seed"), "manifest": m} for m in manifests]})


def validate_curated(doc: dict, where: str = "<curated>") -> list:
    """Problems of a curated multi-seed manifest; each run's manifest is checked with `validate_manifest`."""
    if not isinstance(doc, dict):
        return [f"{where}: must be an object"]
    errs = []
    missing = [k for k in CURATED_REQUIRED if k not in doc]
    if missing:
        errs.append(f"{where}: missing keys: {missing}")
    runs = doc.get("runs")
    if not isinstance(runs, list) or not runs:
        errs.append(f"{where}: runs must be a non-empty array")
        return errs
    for i, r in enumerate(runs):
        if not isinstance(r, dict) or "seed" not in r or "manifest" not in r:
            errs.append(f"{where}: runs[{i}] needs seed and manifest")
            continue
        if isinstance(r["manifest"], dict) and r["manifest"].get("framework") != "pytorch":
            errs.extend(validate_manifest(r["manifest"], f"{where}: runs[{i}].manifest"))
    return errs


def main(argv=None) -> int:
    """python -m rustral_b200.bench.manifest FILE... : validates run or curated manifests, exit 1 on any problem."""
    import argparse
    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("paths", nargs="+")
    a = ap.parse_args(argv)
    bad = 0
    for p in a.paths:
        with open(p, encoding="utf-8") as f:
            doc = json.load(f)
        errs = validate_curated(doc, p) if isinstance(doc, dict) and "runs" in doc else validate_manifest(doc, p)
        for e in errs:
            print(e)
        bad += bool(errs)
    print(f"{'ok' if not bad else 'FAILED'}: validated {len(a.paths)} manifest(s)")
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
