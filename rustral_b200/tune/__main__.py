"""Command line of the autotuner.

    python -m rustral_b200.tune cache                       # what the configuration cache holds
    python -m rustral_b200.tune cache --clear
    python -m rustral_b200.tune gemm --m 32768 --n 2304 --k 768 [--strategy bayesian] [--max-evals 24]
    python -m rustral_b200.tune attention --batch 32 --seq 1024 --heads 12 --head-dim 64
    python -m rustral_b200.tune pretune --model gpt2-small --tokens 32768     # every GEMM shape of a model's step

Tuning needs a GPU (the candidates are timed on it); `cache` and `shapes` work anywhere.  Winners go to the JSON cache
(`$RUSTRAL_CACHE_DIR/autotuner/kernel_configs.json`), from which `GemmTuningTable().apply()` serves them to `ops.gemm`.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from . import AutoTuner, ConfigCache, MatmulShapeBucket, PreTuner, Strategy, TunerConfig, tune_attention, tune_gemm


def _tuner(a) -> AutoTuner:
    cfg = TunerConfig(strategy=Strategy[a.strategy.upper()], max_evals=a.max_evals, max_tuning_time_s=a.max_seconds, verbose=a.verbose)
    return AutoTuner(cfg)


def _need_gpu() -> None:
    if not torch.cuda.is_available():
        raise SystemExit("tuning times the candidates on a GPU; no CUDA device is visible")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="rustral_b200.tune", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p):
        p.add_argument("--strategy", default="bayesian", choices=[s.name.lower() for s in Strategy])
        p.add_argument("--max-evals", type=int, default=24)
        p.add_argument("--max-seconds", type=float, default=30.0)
        p.add_argument("--verbose", action="store_true")
    c = sub.add_parser("cache")
    c.add_argument("--clear", action="store_true")
    c.add_argument("--json", action="store_true", help="print the entries as JSON")
    g = sub.add_parser("gemm")
    for n in ("m", "n", "k"):
        g.add_argument(f"--{n}", type=int, required=True)
    common(g)
    t = sub.add_parser("attention")
    t.add_argument("--batch", type=int, default=32)
    t.add_argument("--seq", type=int, default=1024)
    t.add_argument("--heads", type=int, default=12)
    t.add_argument("--kv-heads", type=int, default=0)
    t.add_argument("--head-dim", type=int, default=64)
    common(t)
    s = sub.add_parser("shapes", help="the GEMM shapes `pretune` would time")
    p = sub.add_parser("pretune")
    for q in (s, p):
        q.add_argument("--model", default="gpt2-small")
        q.add_argument("--tokens", type=int, default=32768)
    common(p)
    a = ap.parse_args(argv)

    if a.cmd == "cache":
        cache = ConfigCache()
        if a.clear:
            cache.entries.clear()
            cache.save()
        if a.json:
            print(json.dumps({k: e.__dict__ for k, e in cache.entries.items()}, indent=1))
        else:
            cache.stats().print()
        return 0
    if a.cmd == "shapes":
        from ..models.config import preset
        for m, n, k in PreTuner().shapes_for(preset(a.model), a.tokens):
            print(f"{m} x {n} x {k}   bucket {MatmulShapeBucket.of(m, n, k).cache_key()}")
        return 0
    _need_gpu()
    tuner = _tuner(a)
    if a.cmd == "gemm":
        r = tune_gemm(a.m, a.n, a.k, tuner)
        print(json.dumps({"shape": [a.m, a.n, a.k], "config": r.config, "time_us": r.time_us, "default_time_us": r.default_time_us,
                          "improvement_pct": r.improvement_pct, "evaluated": r.evaluated, "from_cache": r.from_cache}))
    elif a.cmd == "attention":
        r = tune_attention(a.batch, a.seq, a.heads, a.kv_heads or a.heads, a.head_dim, tuner)
        print(json.dumps({"config": r.config, "time_us": r.time_us, "default_time_us": r.default_time_us, "evaluated": r.evaluated}))
    else:
        from ..models.config import preset
        for shape, r in PreTuner(tuner).pretune(preset(a.model), a.tokens).items():
            print(f"{shape}: {r.config}  {r.time_us:.1f} us (default {r.default_time_us:.1f} us, {r.improvement_pct:+.1f} %)")
    tuner.stats.print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
