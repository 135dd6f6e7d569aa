#!/usr/bin/env python
"""Headline benchmark: training throughput of a GPT-2-small-shaped decoder in bf16 (fp32 master weights, AdamW),
global batch 256 sequences of 1024 tokens, data-parallel with ZeRO sharding across N GPUs of one node.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29501 \
        bench.py --gpus 8 --steps 5 --warmup 3

Two timed regions of `steps` optimizer steps each, both after `warmup` untimed steps:
  * device-timed: token ids already on the device, CUDA events around the steps (max over ranks) -> "value";
  * end to end through the public API (LMTrainer.step): every step copies that step's token ids from pinned host
    memory and reads the loss back to the host -> "e2e".
Rank 0 prints one JSON line.  `--impl reference` reports that the reference cannot be run here.  `--impl torch` runs
the same model, batch and optimizer in plain PyTorch (baseline/torch_gpt2.py: cuBLAS, SDPA, fused AdamW, FSDP) and
prints the same line for it; the framework's own run ends with a short run of that arm on the same GPUs and reports
`vs_baseline` = own tokens/s / its tokens/s (`--no-baseline` skips it).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--zero-stage", type=int, default=3, choices=[2, 3])
    ap.add_argument("--no-baseline", action="store_true", help="skip the plain-PyTorch run behind vs_baseline")
    ap.add_argument("--baseline-steps", type=int, default=0, help="timed steps of the plain-PyTorch run (default: min(steps, 5))")
    ap.add_argument("--model", default="gpt2-small")
    ap.add_argument("--global-batch", type=int, default=256)
    ap.add_argument("--micro-batch", type=int, default=32)
    ap.add_argument("--comm", default="auto", choices=["auto", "nccl", "fused"])
    ap.add_argument("--seq-len", type=int, default=0, help="override the preset's sequence length (tests only)")
    ap.add_argument("--layers", type=int, default=0, help="override the preset's depth (tests only)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, maxc, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                maxc.append(float(parts[2]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxc) if maxc else None, "reasons": sorted(reasons), "samples": len(clocks)}


def reference_arm(args):
    # The reference is a Rust workspace (Cargo.toml, no setup.py / pyproject.toml): `pip install` refuses it, and
    # neither cargo nor rustc exists in this image, so none of its code can be built or run here.
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference is a Rust workspace: pip reports 'not installable, neither setup.py nor "
                                     "pyproject.toml found', and no cargo/rustc toolchain is present to build it"}))
    return 0


def run_torch_arm(args, model, device, rank, world, steps, warmup):
    """The plain-PyTorch arm (no code of this framework on its step)."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
    import torch_gpt2
    return torch_gpt2.run(vocab=model.vocab_padded, seq_len=model.seq_len, n_layer=model.n_layer, heads=model.n_head,
                          d_model=model.d_model, ffn=model.ffn_dim, global_batch=args.global_batch,
                          micro_batch=args.micro_batch, steps=steps, warmup=warmup, device=device, rank=rank, world=world)


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    if args.gpus > 1 and "RANK" not in os.environ:
        # launched directly: re-launch one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + (os.getpid() % 400)), os.path.abspath(__file__)]
        cmd += sys.argv[1:]
        return subprocess.call(cmd)

    import torch
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from rustral_b200 import _native
    from rustral_b200.models.config import preset
    from rustral_b200.runtime.lm_trainer import LMTrainer, TrainConfig

    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    overrides = {}
    if args.seq_len:
        overrides["seq_len"] = args.seq_len
    if args.layers:
        overrides["n_layer"] = args.layers
    model = preset(args.model, **overrides)
    if model.arch != "gpt2" and (args.impl == "torch" or not args.no_baseline):
        raise SystemExit("the plain-PyTorch arm covers the GPT-2 family only: pass --no-baseline")
    data_note = "synthetic (uniform random token ids, fresh batch per step; random-init N(0,0.02) weights)"
    l2_note = "no explicit flush: each step streams >10 GB of activations and a fresh batch, far beyond the 126 MB L2"
    if args.impl == "torch":
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        r = run_torch_arm(args, model, device, rank, world, args.steps, args.warmup)
        clocks = sampler.stop() if rank == 0 else None
        if rank == 0:
            tokens = r["tokens_per_step"]
            print(json.dumps({
                "impl": "torch", "metric": "train_tokens_per_s", "value": round(tokens / (r["ms_per_step"] / 1e3), 1),
                "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": round(r["ms_per_step"], 3), "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": data_note,
                "config": {"model": args.model, "global_batch": args.global_batch, "seq_len": model.seq_len,
                           "parallelism": f"dp{world}-fsdp-full-shard" if world > 1 else "single",
                           "micro_batch": r["micro_batch"], "optimizer": "torch.optim.AdamW(fused), fp32 parameters, bf16 autocast, grad clip 1.0",
                           "stack": "nn.Linear (cuBLAS), F.scaled_dot_product_attention, F.cross_entropy, torch FSDP", "l2": l2_note},
                "clocks": clocks,
                "e2e": {"value": round(tokens / (r["e2e_ms_per_step"] / 1e3), 1), "unit": "tokens/s",
                        "ms_per_step": round(r["e2e_ms_per_step"], 3), "h2d_bytes_per_step": r["h2d_bytes_per_step"],
                        "d2h_bytes_per_step": r["d2h_bytes_per_step"]},
                "gpu_launches": 0, "peak_mem_bytes": r["peak_mem_bytes"], "final_loss": round(r["final_loss"], 4)}))
        if world > 1:
            dist.destroy_process_group()
        return 0
    tcfg = TrainConfig(global_batch=args.global_batch, micro_batch=args.micro_batch, comm=args.comm, zero_stage=args.zero_stage)
    trainer = LMTrainer(model, tcfg, device)
    _native.kernels().rb_init()

    local_b, S = trainer.local_batch, model.seq_len
    total_steps = 2 * (args.warmup + args.steps)
    gen = torch.Generator().manual_seed(1234 + rank)
    # synthetic data: token ids i.i.d. uniform, a fresh batch for every step, in pinned host memory
    host_batches = [torch.randint(0, model.vocab_size, (local_b, S + 1), generator=gen, dtype=torch.int64).pin_memory()
                    for _ in range(total_steps)]
    it = iter(host_batches)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- device-timed region
    dev_batches = [next(it).to(device, non_blocking=True) for _ in range(args.warmup + args.steps)]
    torch.cuda.synchronize()
    for i in range(args.warmup):
        trainer.step_device(dev_batches[i])
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _native.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    losses = []
    for i in range(args.steps):
        losses.append(trainer.step_device(dev_batches[args.warmup + i]))
    e1.record()
    barrier()
    launches = _native.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    dev_ms_per_step = float(ms) / args.steps
    final_loss = float(losses[-1])
    del dev_batches

    # ---------------------------------------------------------------- end-to-end region (public API)
    for _ in range(args.warmup):
        trainer.step(next(it))
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        final_loss_e2e = trainer.step(next(it))     # H2D of the batch + D2H of the loss inside
    torch.cuda.synchronize()
    e2e_s = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=device)
    barrier()
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_ms_per_step = float(e2e_s) * 1e3 / args.steps

    bits, where = _native.read_status()
    symm_bytes = trainer.symmetric_bytes()
    peak_mem = torch.cuda.max_memory_allocated(device) + symm_bytes     # peer-mapped buffers bypass torch's allocator
    state_bytes = trainer.state_bytes()
    label = trainer.parallelism
    comm_name = type(trainer.comm).__name__ if trainer.comm is not None else "none"
    # ---------------------------------------------------------------- plain-PyTorch arm on the same GPUs
    baseline = None
    if not args.no_baseline:
        trainer.close()
        del trainer
        torch.cuda.empty_cache()
        try:
            bsteps = args.baseline_steps or min(args.steps, 5)
            r = run_torch_arm(args, model, device, rank, world, bsteps, min(args.warmup, 3))
            baseline = {"impl": "torch", "value": round(args.global_batch * S / (r["ms_per_step"] / 1e3), 1),
                        "ms_per_step": round(r["ms_per_step"], 3), "steps": bsteps,
                        "e2e_value": round(args.global_batch * S / (r["e2e_ms_per_step"] / 1e3), 1),
                        "peak_mem_bytes": r["peak_mem_bytes"]}
        except Exception as e:      # noqa: BLE001 - the framework's own number must still be printed
            baseline = {"impl": "torch", "failed": f"{type(e).__name__}: {e}"[:300]}
    tokens = args.global_batch * S
    value = tokens / (dev_ms_per_step / 1e3)
    e2e_value = tokens / (e2e_ms_per_step / 1e3)
    if rank == 0:
        flops = model.flops_per_token() * tokens
        ratio = round(value / baseline["value"], 4) if baseline and "value" in baseline else None
        out = {
            "metric": "train_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_ms_per_step, 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": ratio, "baseline": baseline, "dtype": "bf16",
            "data": data_note,
            "config": {"model": args.model, "global_batch": args.global_batch, "seq_len": S,
                       "parallelism": label, "zero_stage": tcfg.zero_stage if world > 1 else None,
                       "micro_batch": min(args.micro_batch, local_b), "optimizer": "AdamW, fp32 master weights, grad clip 1.0",
                       "comm": comm_name, "layers": model.n_layer, "d_model": model.d_model,
                       "vocab": model.vocab_size, "vocab_padded": model.vocab_padded,
                       "l2": l2_note},
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms_per_step, 3),
                    "h2d_bytes_per_step": local_b * (S + 1) * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "peak_mem_bytes": peak_mem, "symmetric_bytes": symm_bytes, "state_bytes": state_bytes,
            "model_tflops_per_s": round(flops / (dev_ms_per_step / 1e3) / 1e12, 1),
            "final_loss": round(final_loss, 4), "final_loss_e2e": round(final_loss_e2e, 4),
            "device_status": bits,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
