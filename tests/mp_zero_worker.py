"""Worker for the multi-rank ZeRO tests: launched with torch.distributed.run, one rank per device (or CPU/gloo).

Trains a small decoder for a few steps with the requested communicator and prints, on rank 0, one JSON line with
the losses and a checksum of the final parameters so that the parent test can compare configurations.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--comm", default="nccl")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--model", default="gpt2-test")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--zero-stage", type=int, default=3)
    ap.add_argument("--reopen", action="store_true",
                    help="close the trainer, build a second one in the same process and step it (peer tables must not be reused)")
    ap.add_argument("--resume-check", action="store_true",
                    help="snapshot weights + per-rank optimizer state, resume in a second trainer, compare the next steps")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if a.device == "cuda":
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    from rustral_b200 import _native
    from rustral_b200.models.config import preset
    from rustral_b200.runtime.lm_trainer import LMTrainer, TrainConfig
    cfg = preset(a.model, **({"n_layer": a.layers} if a.layers else {}))
    tcfg = lambda: TrainConfig(global_batch=8, micro_batch=2, lr=1e-3, comm=a.comm, zero_stage=a.zero_stage)
    tr = LMTrainer(cfg, tcfg(), dev)
    g = torch.Generator().manual_seed(7)
    data = torch.randint(0, cfg.vocab_size, (8, cfg.seq_len + 1), generator=g, dtype=torch.int64)
    local = data[rank * tr.local_batch:(rank + 1) * tr.local_batch].contiguous()
    if a.device == "cuda":
        local = local.pin_memory()
    losses = [tr.step(local) for _ in range(a.steps)]
    sd = tr.state_dict()
    checksum = float(sum(v.double().abs().sum() for v in sd.values()))
    probe = sd["layers.0.attn.wq.weight"].flatten()[:8].tolist()
    status = 0
    if a.device == "cuda":
        torch.cuda.synchronize()
        status = _native.read_status()[0]
    resume = None
    if a.resume_check:
        opt_tensors, opt_meta = tr.optimizer_state()
        tr2 = LMTrainer(cfg, tcfg(), dev)
        tr2.load_state_dict(sd)
        tr2.load_optimizer_state(opt_tensors, opt_meta)
        cont = [tr.step(local) for _ in range(2)]
        again = [tr2.step(local) for _ in range(2)]
        resume = {"continued": cont, "resumed": again, "shard_len": opt_meta["shard_len"], "world": opt_meta["world"],
                  "moments_numel": int(opt_tensors["adam.m"].numel())}
        tr2.close()
    comm_name = type(tr.comm).__name__ if tr.comm is not None else "none"
    label, state_bytes = tr.parallelism, tr.state_bytes()
    reopened = None
    if a.reopen:
        tr.close()
        tr = LMTrainer(cfg, tcfg(), dev)              # same process, new symmetric buffers and peer tables
        reopened = [tr.step(local) for _ in range(a.steps)]
        if a.device == "cuda":
            torch.cuda.synchronize()
            status |= _native.read_status()[0]
    if rank == 0:
        print(json.dumps({"losses": losses, "checksum": checksum, "probe": probe, "status": status, "resume": resume,
                          "comm": comm_name, "parallelism": label, "state_bytes": state_bytes, "reopened": reopened}))
    tr.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
