"""Data-parallel training across processes on the CPU: each rank takes its share of every batch, gradients are averaged
over the `gloo` backend, and every rank ends with bit-identical parameters.  Started without a launcher it spawns its own
ranks; under `torchrun` it uses the ranks it is given (crates/distributed/examples/mpi_dp_cpu.rs runs the same experiment
under `mpirun -n 4`).

    python examples/dp_cpu_gloo.py [--world 2] [--steps 30] [--overlap]
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29517 examples/dp_cpu_gloo.py
"""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from _common import parser

from rustral_b200.core import CpuBackend, ForwardCtx
from rustral_b200.nn import LinearBuilder, MSELoss, Sequential
from rustral_b200.optim import Adam
from rustral_b200.parallel.data_parallel import DataParallelTrainer
from rustral_b200.parallel.process_group import ProcessGroup


def worker(rank, world, a, port, out):
    if world > 1 and not dist.is_initialized():
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        dist.init_process_group("gloo", rank=rank, world_size=world)
    pg = ProcessGroup.from_torch() if world > 1 else ProcessGroup.new_single_process()
    backend = CpuBackend()
    model = Sequential(LinearBuilder(8, 32).with_bias().seed(a.seed).activation("relu").build(backend),
                       LinearBuilder(32, 1).with_bias().seed(a.seed + 1).build(backend))
    g = torch.Generator().manual_seed(a.seed)                      # every rank draws the same global batches
    w_true = torch.randn(8, 1, generator=g)
    trainer = DataParallelTrainer(pg, Adam(lr=1e-2), overlap=a.overlap)
    mse = MSELoss()

    def loss_fn(local, ctx):
        x = torch.stack([s[0] for s in local])
        y = torch.stack([s[1] for s in local])
        return mse(model(x, ctx), y)
    losses = []
    for _ in range(a.steps):
        x = torch.randn(32, 8, generator=g)
        batch = list(zip(x, x @ w_true))
        losses.append(trainer.step(model.parameters(), batch, loss_fn, ForwardCtx.train(backend)))
    digest = float(sum(p.tensor.detach().double().sum() for p in model.parameters()))
    digests = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
    if world > 1:
        dist.all_gather(digests, torch.tensor([digest], dtype=torch.float64))
    else:
        digests[0][0] = digest
    if rank == 0:
        same = all(float(d) == float(digests[0]) for d in digests)
        print(f"{world} rank(s): global loss {losses[0]:.4f} -> {losses[-1]:.4f}; parameters identical on every rank: {same}")
        if out is not None:
            out.update(loss_first=losses[0], loss_last=losses[-1], identical=same, world=world)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _spawned(rank, world, a, port, q):
    out = {} if rank == 0 else None
    worker(rank, world, a, port, out)
    if rank == 0:
        q.put(out)


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--overlap", action="store_true", help="reduce gradient buckets during the backward pass")
    ap.add_argument("--port", type=int, default=29517)
    a = ap.parse_args(argv)
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:        # started by torchrun
        dist.init_process_group("gloo")
        out = {}
        worker(dist.get_rank(), dist.get_world_size(), a, a.port, out)
        return out
    if a.world == 1:
        out = {}
        worker(0, 1, a, a.port, out)
        return out
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_spawned, args=(r, a.world, a, a.port, q)) for r in range(a.world)]
    for p in procs:
        p.start()
    out = q.get()
    for p in procs:
        p.join()
    if any(p.exitcode for p in procs):
        sys.exit("a rank failed")
    return out


if __name__ == "__main__":
    main()
