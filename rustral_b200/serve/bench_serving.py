"""Serving benchmark: Poisson arrivals against the continuous-batching engine; prints one JSON line with p50/p99 TTFT,
inter-token latency and output tokens/s.

    python -m rustral_b200.serve.bench_serving --model llama-8b --layers 4 --requests 64 --rate 8
"""
from __future__ import annotations

import argparse
import json

import torch

from ..models.config import preset
from .engine import ServingEngine, run_poisson_workload
from .model_runner import ModelRunner


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-8b")
    ap.add_argument("--layers", type=int, default=0, help="override depth (a full 8B model needs ~16 GB of weights)")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--rate", type=float, default=8.0)
    ap.add_argument("--prompt", type=int, nargs=2, default=[128, 2048])
    ap.add_argument("--output", type=int, nargs=2, default=[128, 512])
    ap.add_argument("--max-batch", type=int, default=64)
    ap.add_argument("--blocks", type=int, default=16384)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    over = {"n_layer": a.layers} if a.layers else {}
    cfg = preset(a.model, **over)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    runner = ModelRunner(cfg, device=dev, num_blocks=a.blocks, block_size=a.page, seed=a.seed)
    eng = ServingEngine(runner, max_batch_size=a.max_batch)
    # warm-up: one short request end to end
    eng.generate(list(range(1, 33)), 4)
    eng.scheduler.completed.clear()
    m = run_poisson_workload(eng, a.requests, a.rate, tuple(a.prompt), tuple(a.output), a.seed)
    out = {"metric": "serving", "model": a.model, "layers": cfg.n_layer, "requests": a.requests, "rate_per_s": a.rate,
           "page_size": a.page, "decoding": "greedy", "data": "synthetic uniform random prompt tokens; random-init weights"}
    out.update(m.to_dict())
    print(json.dumps(out))


if __name__ == "__main__":
    main()
