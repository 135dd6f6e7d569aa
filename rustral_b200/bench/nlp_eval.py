"""Multi-seed NLP evaluation: runs the SST-2 and WikiText-2 examples once per seed and curates the run manifests into
one JSON per task with mean / std aggregates (scripts/eval/run_nlp_real.py).

    python -m rustral_b200.bench.nlp_eval --benchmark --seeds 0,1,2 --out benchmarks/runs/v0.1.0/nlp
    python -m rustral_b200.bench.nlp_eval --paper --tasks sst2 --device cuda:0

`--benchmark` is the fast preset (the examples' `--quick` mode with a one-layer model); `--paper` the large one.  The
datasets come from the cache (`RUSTRAL_CACHE_DIR`); with `RUSTRAL_DATASET_OFFLINE=1` nothing is downloaded.  The
vocabulary fitted by the first seed is reused by the others, so that every seed trains the same model shape.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import shutil
import sys

from .manifest import curate, validate_curated

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
TASKS = {"sst2": ("sst2_classifier", "sst2_classifier", "dev_accuracy"),
         "wikitext2": ("wikitext2_lm", "wikitext2_word_lm", "dev_perplexity")}


def _example(name: str):
    path = os.path.join(ROOT, "examples", name + ".py")
    spec = importlib.util.spec_from_file_location(f"rustral_example_{name}", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def run_task(task: str, seeds, out_dir: str, preset: str, device: str = "cpu", extra=()) -> dict:
    """Runs `task` for every seed (per-seed outputs under `<out_dir>/raw/<task>/seed<N>`), writes
    `<out_dir>/<task>.json` and returns the curated document."""
    example, task_name, metric = TASKS[task]
    mod = _example(example)
    manifests, vocab = [], None
    for seed in seeds:
        run_dir = os.path.join(out_dir, "raw", task, f"seed{seed}")
        os.makedirs(run_dir, exist_ok=True)
        args = ["--seed", str(seed), "--out-dir", run_dir, "--device", device, *extra]
        if preset == "benchmark":
            args += ["--quick", "--num-layers", "1", "--d-model", "32", "--num-heads", "2", "--ffn-dim", "64"]
            args += ["--block-size", "16"] if task == "wikitext2" else ["--seq-len", "16"]
        elif preset == "paper":
            args += ["--paper"]
        if task == "sst2" and vocab is not None:
            args += ["--vocab", vocab]
        manifests.append(mod.main(args))
        if vocab is None and os.path.exists(os.path.join(run_dir, "vocab.txt")):
            vocab = os.path.join(run_dir, "vocab.txt")
    doc = curate(task_name, metric, os.environ.get("RUSTRAL_EVAL_VERSION", "0.1.0"), manifests)
    problems = validate_curated(doc, task)
    if problems:
        raise SystemExit("\n".join(problems))
    path = os.path.join(out_dir, f"{task}.json")
    with open(path + ".tmp", "w", encoding="utf-8") as f:
        json.dump(doc, f, indent=2)
        f.write("\n")
    os.replace(path + ".tmp", path)
    return doc


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="rustral_b200.bench.nlp_eval", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--seeds", default="0,1,2", help="comma-separated list")
    ap.add_argument("--tasks", default="sst2,wikitext2")
    ap.add_argument("--benchmark", action="store_true", help="fast preset: tiny model, quick data caps")
    ap.add_argument("--paper", action="store_true", help="large preset")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--out", default=os.path.join("benchmarks", "runs", "v0.1.0", "nlp"))
    ap.add_argument("--clean", action="store_true", help="remove the output directory first")
    a = ap.parse_args(argv)
    if a.benchmark and a.paper:
        raise SystemExit("--benchmark and --paper exclude each other")
    seeds = [int(s) for s in a.seeds.split(",") if s.strip()]
    if not seeds:
        raise SystemExit("no seeds")
    if a.clean and os.path.isdir(a.out):
        shutil.rmtree(a.out)
    os.makedirs(a.out, exist_ok=True)
    preset = "benchmark" if a.benchmark else "paper" if a.paper else "default"
    for task in [t.strip() for t in a.tasks.split(",") if t.strip()]:
        if task not in TASKS:
            raise SystemExit(f"unknown task {task}; choose from {sorted(TASKS)}")
        doc = run_task(task, seeds, a.out, preset, a.device)
        agg = doc["aggregate"]
        print(f"{task}: {doc['metric']} mean={agg['mean']:.4f} std={agg['std']:.4f} over {agg['n']} seed(s) -> "
              f"{os.path.join(a.out, task + '.json')}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
