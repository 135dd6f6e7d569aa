"""Serving benchmark: Poisson arrivals against the continuous-batching engine; prints one JSON line with p50/p99 TTFT,
inter-token latency and output tokens/s.

    python -m rustral_b200.serve.bench_serving --model llama-8b --layers 4 --requests 64 --rate 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29720 \
        -m rustral_b200.serve.bench_serving --model llama-8b --tp 8 --requests 2000 --rate 8
    python -m rustral_b200.serve.bench_serving --model llama-8b --layers 8 --requests 300 --rates 8 16 32 64

`--rates` runs the workload once per arrival rate (ascending) and stops after the first rate whose p99 time to first
token exceeds `--ttft-limit-ms`: below that point tokens/s follows the offered load, at it the engine is saturated and
tokens/s is its capacity.  `--prefill-chunk` is the number of prompt tokens a step processes besides its decode batch.

With `--tp N` every rank runs the same engine on its shard of the model (one-shot peer-memory all-reduce after the
attention-output and down projections, all-gather of the vocabulary-sharded logits); rank 0's clock decides when a
request has arrived, so the ranks stay in lockstep, and rank 0 prints the result.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

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
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--time-limit", type=float, default=3600.0)
    ap.add_argument("--rates", type=float, nargs="+", default=None, help="arrival-rate sweep (requests/s), ascending")
    ap.add_argument("--ttft-limit-ms", type=float, default=1000.0, help="the sweep stops once p99 TTFT exceeds this")
    ap.add_argument("--tp-allreduce", default=None, choices=["peer", "nvls"],
                    help="per-layer all-reduce of the tensor-parallel ranks: peer loads (default) or in-switch multimem reduction")
    ap.add_argument("--prefill-chunk", type=int, default=2048, help="prompt tokens per step (0: whole prompts, one pass each)")
    a = ap.parse_args(argv)
    over = {"n_layer": a.layers} if a.layers else {}
    cfg = preset(a.model, **over)
    rank = 0
    tp = clock = None
    if a.tp > 1:
        rank = int(os.environ["RANK"])
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
        if dist.get_world_size() != a.tp:
            raise SystemExit(f"--tp {a.tp} but WORLD_SIZE={dist.get_world_size()}")
        from ..parallel.tp_inference import TPInferenceComm
        rows = max(a.prompt[1], a.max_batch, a.prefill_chunk + a.max_batch)
        tp = TPInferenceComm(None, dev, max_elems=rows * max(cfg.d_model, cfg.vocab_padded // a.tp), transport=a.tp_allreduce)
        clock = tp.broadcast_scalar
    else:
        dev = "cuda" if torch.cuda.is_available() else "cpu"
    if tp is None and cfg.arch == "llama" and str(dev) != "cpu":
        from .weights import InferenceWeights           # bf16 weights only: the trainer's flat buffers would not fit
        params = InferenceWeights.random_llama(cfg, dev, 0, 1, a.seed)
    else:
        params = None
    runner = ModelRunner(cfg, params=params, device=dev, num_blocks=a.blocks, block_size=a.page, seed=a.seed, tp=tp)
    eng = ServingEngine(runner, max_batch_size=a.max_batch, prefill_chunk=a.prefill_chunk)
    # warm-up: one short request end to end
    eng.generate(list(range(1, 33)), 4)
    eng.scheduler.completed.clear()
    out = {"metric": "serving", "model": a.model, "layers": cfg.n_layer, "requests": a.requests, "rate_per_s": a.rate,
           "page_size": a.page, "decoding": "greedy", "tp": a.tp, "tp_allreduce": (tp.transport if tp is not None else None), "prefill_chunk": a.prefill_chunk, "max_batch": a.max_batch,
           "data": "synthetic uniform random prompt tokens; random-init weights"}
    if a.rates:
        sweep, saturated = [], None
        for rate in sorted(a.rates):
            eng.scheduler.completed.clear()
            m = run_poisson_workload(eng, a.requests, rate, tuple(a.prompt), tuple(a.output), a.seed, a.time_limit, clock)
            row = {"rate_per_s": rate, **m.to_dict()}
            sweep.append(row)
            if m.ttft_p99_ms > a.ttft_limit_ms:
                saturated = rate
                break
        out.update({"sweep": sweep, "saturated_at_rate": saturated,
                    "capacity_tokens_per_s": max(r["output_tokens_per_s"] for r in sweep)})
    else:
        m = run_poisson_workload(eng, a.requests, a.rate, tuple(a.prompt), tuple(a.output), a.seed, a.time_limit, clock)
        out.update(m.to_dict())
    if a.tp > 1:
        from .. import _native
        st = torch.tensor([_native.read_status()[0]], device=dev)
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        out["device_status"] = int(st)
        dist.barrier()
        tp.close()
    if rank == 0:
        print(json.dumps(out))
    if a.tp > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
