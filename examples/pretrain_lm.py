"""Language-model pre-training from a token file: the production path end to end.

Memory-mapped token file -> native prefetcher (pinned buffers, a worker thread ahead of the GPU) -> `LMTrainer`
(hand-scheduled forward / backward, bf16 compute with fp32 master AdamW; with several ranks the ZeRO gradient
reduction + optimizer + parameter push run as peer-memory kernels over NVLink) -> warm-up + cosine learning rate ->
asynchronous checkpoints (weights on rank 0, the Adam moments of every rank's shard, written by the C++ writer pool
while training continues) -> resume that reproduces the uninterrupted run.

    python examples/pretrain_lm.py --model gpt2-small --tokens corpus.bin --steps 1000 --out runs/gpt2
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/pretrain_lm.py \
        --model gpt2-small --tokens corpus.bin --steps 1000 --global-batch 256 --out runs/gpt2
    python examples/pretrain_lm.py ... --resume runs/gpt2          # continues from the last complete checkpoint

Without `--tokens` a synthetic corpus (a noisy periodic sequence) is written into `--out` first.
"""
import argparse
import json
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rustral_b200.data.datasets import TokenFileDataset                       # noqa: E402
from rustral_b200.io import safetensors_io as st                              # noqa: E402
from rustral_b200.metrics import create_logger                                # noqa: E402
from rustral_b200.models.config import preset                                 # noqa: E402
from rustral_b200.optim import WarmupCosine                                   # noqa: E402
from rustral_b200.parallel.checkpoint import AsyncCheckpointWriter            # noqa: E402
from rustral_b200.runtime.lm_trainer import LMTrainer, TrainConfig            # noqa: E402


def synthetic_corpus(path: str, vocab: int, tokens: int = 200_000, seed: int = 0) -> None:
    rng = np.random.default_rng(seed)
    base = (np.arange(tokens) * 7 + (np.arange(tokens) // 13)) % min(vocab, 251)
    noise = rng.integers(0, vocab, tokens)
    out = np.where(rng.random(tokens) < 0.1, noise, base).astype(np.uint16 if vocab <= 65536 else np.int32)
    out.tofile(path)


def latest_checkpoint(out_dir: str):
    """The newest step directory that has its `complete.json` marker (written last, after every rank's files)."""
    best = None
    for name in os.listdir(out_dir) if os.path.isdir(out_dir) else []:
        if name.startswith("step_") and os.path.exists(os.path.join(out_dir, name, "complete.json")):
            n = int(name[5:])
            best = n if best is None or n > best else best
    return best


def queue_checkpoint(trainer, writer, out_dir: str, step: int, rank: int) -> str:
    """Snapshots this rank's state into host memory and queues its files on the writer pool; returns at once, so the
    next training steps run while the disk is written.  `publish_checkpoint` makes it count."""
    d = os.path.join(out_dir, f"step_{step}")
    os.makedirs(d, exist_ok=True)
    weights = trainer.state_dict()                                   # collective: gathers the fp32 master shards
    opt_tensors, opt_meta = trainer.optimizer_state()
    if rank == 0:
        writer.write(os.path.join(d, "model.safetensors"), st.serialize(weights, {"step": str(step)}))
    writer.write(os.path.join(d, f"optimizer_rank_{rank}.safetensors"),
                 st.serialize(opt_tensors, {k: str(v) for k, v in opt_meta.items()}))
    return d


def publish_checkpoint(writer, d: str, step: int, rank: int, world: int, barrier) -> None:
    """Collective: waits for every rank's queued files, then rank 0 writes the `complete.json` marker."""
    writer.flush()
    barrier()
    if rank == 0:
        with open(os.path.join(d, "complete.json.partial"), "w") as f:
            json.dump({"step": step, "world": world, "time": time.time()}, f)
        os.replace(os.path.join(d, "complete.json.partial"), os.path.join(d, "complete.json"))
    barrier()


def load_checkpoint(trainer, out_dir: str, step: int, rank: int) -> None:
    d = os.path.join(out_dir, f"step_{step}")
    weights, _ = st.load_file(os.path.join(d, "model.safetensors"))
    trainer.load_state_dict(weights)
    tensors, meta = st.load_file(os.path.join(d, f"optimizer_rank_{rank}.safetensors"))
    trainer.load_optimizer_state(tensors, {k: int(v) for k, v in meta.items()})


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="gpt2-small")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--seq-len", type=int, default=0)
    ap.add_argument("--d-model", type=int, default=0)
    ap.add_argument("--tokens", help="flat file of token ids (uint16, or int32 with --int32)")
    ap.add_argument("--int32", action="store_true")
    ap.add_argument("--steps", type=int, default=100, help="length of the run (the horizon of the learning-rate schedule)")
    ap.add_argument("--stop-after", type=int, default=0, help="stop at this step (a checkpoint is written); resume later")
    ap.add_argument("--global-batch", type=int, default=32)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--lr", type=float, default=6e-4)
    ap.add_argument("--min-lr", type=float, default=6e-5)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--checkpoint-every", type=int, default=50)
    ap.add_argument("--log-every", type=int, default=10)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default=None)
    ap.add_argument("--out", default="runs/pretrain")
    ap.add_argument("--resume", action="store_true", help="continue from the newest complete checkpoint in --out")
    a = ap.parse_args(argv)

    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    device = a.device or (f"cuda:{os.environ.get('LOCAL_RANK', 0)}" if torch.cuda.is_available() else "cpu")
    if world > 1:
        import torch.distributed as dist
        if device.startswith("cuda"):
            torch.cuda.set_device(torch.device(device))
            dist.init_process_group("nccl", device_id=torch.device(device))
        else:
            dist.init_process_group("gloo")
        barrier = dist.barrier
    else:
        barrier = lambda: None
    over = {k: v for k, v in (("n_layer", a.layers), ("seq_len", a.seq_len), ("d_model", a.d_model)) if v}
    cfg = preset(a.model, **over)
    os.makedirs(a.out, exist_ok=True)
    tokens = a.tokens
    if not tokens:
        tokens = os.path.join(a.out, "synthetic_tokens.bin")
        if rank == 0 and not os.path.exists(tokens):
            synthetic_corpus(tokens, cfg.vocab_size, seed=a.seed)
        barrier()
    data = TokenFileDataset(tokens, cfg.seq_len, 4 if (a.int32 or (not a.tokens and cfg.vocab_size > 65536)) else 2,
                            seed=a.seed * 1000 + rank)               # every rank draws its own windows
    trainer = LMTrainer(cfg, TrainConfig(global_batch=a.global_batch, micro_batch=a.micro_batch, lr=a.lr, seed=a.seed), device)
    schedule = WarmupCosine(a.lr, a.min_lr, a.warmup, a.steps)
    first = 0
    if a.resume:
        last = latest_checkpoint(a.out)
        if last is not None:
            load_checkpoint(trainer, a.out, last, rank)
            first = last
            if rank == 0:
                print(f"resumed from step {last}")
    logger = create_logger(a.out, "pretrain", console=False) if rank == 0 else None
    writer = AsyncCheckpointWriter()
    losses, t0, tok_per_step = [], time.perf_counter(), a.global_batch * cfg.seq_len

    def on_step(step, loss):
        losses.append(loss)
        n = step + 1
        if logger is not None:
            logger.log_scalar_with_step("train/loss", loss, step)
            logger.log_scalar_with_step("train/lr", schedule.get_lr(step), step)
            if n % a.log_every == 0 or n == end:
                dt = time.perf_counter() - t0
                print(f"[step {n}] loss={loss:.4f} lr={schedule.get_lr(step):.2e} {(n - first) * tok_per_step / dt:,.0f} tokens/s")

    step, pending = first, None
    end = min(a.steps, a.stop_after) if a.stop_after > 0 else a.steps
    while step < end:
        upto = min(end, (step // a.checkpoint_every + 1) * a.checkpoint_every) if a.checkpoint_every > 0 else end
        trainer.fit_token_file(data, upto - step, first_step=step, lr_schedule=schedule.get_lr, on_step=on_step)
        step = upto
        if a.checkpoint_every > 0 and (step % a.checkpoint_every == 0 or step == end):
            if pending is not None:                                  # the previous checkpoint was written under the last steps
                publish_checkpoint(writer, *pending, rank, world, barrier)
            pending = (queue_checkpoint(trainer, writer, a.out, step, rank), step)
    if pending is not None:
        publish_checkpoint(writer, *pending, rank, world, barrier)
    writer.close()
    if logger is not None:
        logger.flush()
    summary = {"model": a.model, "steps": a.steps, "first_step": first, "world": world, "loss_first": losses[0] if losses else None,
               "loss_last": losses[-1] if losses else None, "losses": losses,
               "tokens_per_s": (end - first) * tok_per_step / max(1e-9, time.perf_counter() - t0),
               "last_checkpoint": latest_checkpoint(a.out)}
    if rank == 0:
        with open(os.path.join(a.out, "summary.json"), "w") as f:
            json.dump(summary, f, indent=1)
    trainer.close()
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return summary


if __name__ == "__main__":
    main()
