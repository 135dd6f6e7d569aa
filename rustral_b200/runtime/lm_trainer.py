"""Public training entry point for decoder-only language models: ``LMTrainer``.

One process per GPU.  A step takes a pinned host tensor of token ids [local_batch, seq_len + 1], copies it to the
device, runs the fused engine over micro-batches, reduces gradients across data-parallel ranks (ZeRO: gradients
reduce-scattered, optimizer state and master weights sharded, bf16 parameters gathered), applies AdamW and returns
the mean loss as a Python float (one device-to-host read per step).

Replaces the reference's TapeTrainer / DataParallelTrainer / FSDP.train_step stack
(crates/runtime/src/tape_trainer.rs:296-485, crates/distributed/src/lib.rs:330-412, crates/distributed/src/fsdp.rs:362-386).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from .. import ops
from ..models.config import GPTConfig
from .fused_gpt import ALIGN, FusedGPTEngine


@dataclass
class TrainConfig:
    global_batch: int = 256          # sequences per optimizer step over all ranks
    micro_batch: int = 32            # sequences per forward/backward pass on one rank
    lr: float = 3e-4
    betas: tuple = (0.9, 0.95)
    eps: float = 1e-8
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    seed: int = 0
    # How the data-parallel ranks share the training state (one rank: everything is local, the stage is moot):
    #   3: parameters, gradients and optimizer state sharded; each block's parameters are gathered just before it runs
    #      (forward and backward) and its gradients reduce-scattered right after its backward, overlapped with compute
    #      (parallel/zero3.py);
    #   2: optimizer state and the gradient reduction sharded, every rank keeps a full bf16 working copy and a full
    #      fp32 gradient buffer; the owner pushes updated parameters into every rank's copy after the step
    #      (parallel/fused_zero.py, or library collectives in parallel/zero_comm.py).
    zero_stage: int = 3
    comm: str = "auto"               # "nccl": library collectives; "fused": peer-memory kernels; "auto": fused on CUDA devices


class LMTrainer:
    def __init__(self, model: GPTConfig, train: TrainConfig | None = None, device=None, process_group=None):
        self.model_cfg = model
        self.cfg = train or TrainConfig()
        if device is None:
            device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        if self.device.type == "cuda":
            if self.device.index is None:
                self.device = torch.device("cuda", torch.cuda.current_device())
            torch.cuda.set_device(self.device)
        self.pg = process_group
        self.world = 1
        self.rank = 0
        if process_group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()):
            self.world = torch.distributed.get_world_size(process_group)
            self.rank = torch.distributed.get_rank(process_group)
        c = self.cfg
        if c.global_batch % self.world:
            raise ValueError("global_batch must be divisible by the number of ranks")
        self.local_batch = c.global_batch // self.world
        self.micro_batch = min(c.micro_batch, self.local_batch)
        if self.local_batch % self.micro_batch:
            raise ValueError("the per-rank batch must be a multiple of the micro-batch")
        if c.zero_stage not in (2, 3):
            raise ValueError("zero_stage must be 2 or 3")
        self.zero_stage = c.zero_stage if self.world > 1 else 0
        store = None
        if self.zero_stage == 3:
            from ..parallel.zero3 import ShardedParams
            peer = self.device.type == "cuda" and c.comm in ("auto", "fused")
            if c.comm == "fused" and not peer:
                raise ValueError("the fused ZeRO kernels need CUDA devices")
            store = ShardedParams(model, self.device, c.seed, group=process_group, transport="peer" if peer else "collective")
        self.engine = FusedGPTEngine(model, self.device, self.micro_batch, c.seed, c.lr, c.betas, c.eps, c.weight_decay,
                                     c.max_grad_norm, flat_pad_to=ALIGN * self.world, params=store)
        if store is not None and not store.transport.overlapped:
            self.engine.use_graphs = False           # library collectives are issued eagerly
        self.tokens_per_step = c.global_batch * model.seq_len
        P = self.engine.params
        if store is not None:
            self.shard_len = P.shard_len
            self.shard = slice(self.rank * P.shard_len, (self.rank + 1) * P.shard_len)   # position in rank-major order
        else:
            self.shard_len = P.total // self.world
            self.shard = slice(self.rank * self.shard_len, (self.rank + 1) * self.shard_len)
        self._dev_tokens = None
        self._loss_host = torch.zeros((), dtype=torch.float32).pin_memory() if self.device.type == "cuda" else None
        self._norm_buf = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._grad_lowp = None
        self.comm = None
        if self.zero_stage == 3:
            from ..parallel.zero3 import Zero3Comm
            self.comm = Zero3Comm(self)
        elif self.world > 1:
            from ..parallel.zero_comm import make_zero_comm
            self.comm = make_zero_comm(self, c.comm)

    @property
    def parallelism(self) -> str:
        """Truthful label of how the ranks share the state, e.g. "dp8-zero3-peer", "dp8-zero2-push", "single"."""
        if self.world == 1:
            return "single"
        kind = type(self.comm).__name__
        tr = getattr(self.engine.params, "transport", None)
        peer = "peer-nvls" if getattr(tr, "reduce_mode", "") == "nvls" else "peer"
        how = {"Zero3Comm": peer if getattr(tr, "overlapped", False) else "collective",
               "FusedZeroComm": "push", "NcclZeroComm": "nccl"}.get(kind, kind)
        return f"dp{self.world}-zero{self.zero_stage}-{how}"

    def symmetric_bytes(self) -> int:
        """Bytes this rank holds in peer-mapped buffers; they come from the driver directly, not from torch's
        allocator, so torch's memory statistics do not count them."""
        owner = getattr(self.engine.params, "transport", None) if self.zero_stage == 3 else self.comm
        bufs = getattr(owner, "_symm", None)
        if bufs is None and owner is not None:
            bufs = [getattr(owner, n) for n in ("grad_buf", "lowp_buf", "norm_buf", "pad") if hasattr(owner, n)]
        return int(sum(getattr(b, "nbytes", 0) for b in (bufs or [])))

    def state_bytes(self) -> dict:
        """Bytes of parameters, gradients and optimizer state held by THIS rank (activations excluded)."""
        P = self.engine.params
        if self.zero_stage == 3:
            return P.state_bytes()
        lp = P.lowp.element_size()
        if self.comm is not None and hasattr(self.comm, "master"):      # stage 2 over peer memory
            return {"param_full": P.total * lp, "grad_full": P.total * 4, "optimizer_shard": 3 * self.shard_len * 4,
                    "grad_shard": self.shard_len * 4, "unsharded_leftover": 3 * P.total * 4}
        return {"param_full": P.total * lp, "grad_full": P.total * 4, "optimizer_full": 3 * P.total * 4}

    # -------------------------------------------------------------------------------------------------
    def step_device(self, tokens_dev: torch.Tensor, lr: float | None = None) -> torch.Tensor:
        """tokens_dev: int64 [local_batch, seq_len + 1] already on the device.  Returns the loss as a device scalar."""
        eng = self.engine
        ids = tokens_dev[:, :-1]
        tgt = tokens_dev[:, 1:]
        if not ids.is_contiguous():
            ids, tgt = ids.contiguous(), tgt.contiguous()
        loss = eng.train_step(ids, tgt, total_tokens=self.tokens_per_step, lr=lr, do_step=(self.world == 1))
        if self.zero_stage == 3:
            loss = self.comm.reduce_and_step(eng.loss_acc, lr)       # the summed token loss; the exchange scales it
        elif self.world > 1:
            loss = self.comm.reduce_and_step(loss, lr)
        return loss

    def step(self, tokens_host: torch.Tensor, lr: float | None = None) -> float:
        """tokens_host: int64 [local_batch, seq_len + 1] in (preferably pinned) host memory.  Returns the mean loss."""
        if self.device.type == "cuda":
            if self._dev_tokens is None or self._dev_tokens.shape != tokens_host.shape:
                self._dev_tokens = torch.empty(tokens_host.shape, dtype=torch.int64, device=self.device)
            self._dev_tokens.copy_(tokens_host, non_blocking=True)
            loss = self.step_device(self._dev_tokens, lr)
            self._loss_host.copy_(loss, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return float(self._loss_host)
        return float(self.step_device(tokens_host, lr))

    def fit_token_file(self, dataset, steps: int, first_step: int = 0, lr_schedule=None, on_step=None, depth: int = 3) -> list:
        """Trains `steps` optimizer steps on a `data.TokenFileDataset`: a native worker thread gathers the windows of
        the coming steps into pinned buffers while the GPU works on the current one.  With several ranks every rank
        passes a dataset with its own seed, so that the ranks draw different windows.  `lr_schedule(step) -> lr`,
        `on_step(step, loss)`.  Returns the losses.  Resuming at `first_step` reproduces the data of an uninterrupted run."""
        if dataset.seq_len != self.model_cfg.seq_len:
            raise ValueError(f"the dataset serves windows of {dataset.seq_len} tokens, the model takes {self.model_cfg.seq_len}")
        pf = dataset.prefetcher(self.local_batch, depth, first_step)
        losses = []
        try:
            for _ in range(steps):
                tokens, s = pf.next()
                loss = self.step(tokens, lr_schedule(s) if lr_schedule is not None else None)
                losses.append(loss)
                if on_step is not None:
                    on_step(s, loss)
        finally:
            pf.close()
        return losses

    # -------------------------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        if self.comm is not None:
            self.comm.gather_master()
        return self.engine.params.state_dict()

    def close(self) -> None:
        """Releases peer mappings (collective when world > 1)."""
        if self.comm is not None:
            self.comm.close()
            self.comm = None

    def load_state_dict(self, state: dict) -> None:
        self.engine.params.load_state_dict(state)
        if self.comm is not None:
            self.comm.reload_master()

    def optimizer_state(self) -> tuple:
        """(tensors, meta) of THIS rank's optimizer state: the Adam moments of its shard of the flat parameter space
        and the step count.  Together with `state_dict()` it makes a resumed run continue bit for bit; every rank
        saves its own (the layout of `DistributedCheckpointManager`: one file per rank)."""
        if self.comm is not None:
            m, v = self.comm.optimizer_shard()
        else:
            P = self.engine.params
            m, v = P.m, P.v
        tensors = {"adam.m": m.detach().float().cpu().clone(), "adam.v": v.detach().float().cpu().clone()}
        meta = {"step": int(self.engine.step_count), "world": self.world, "rank": self.rank,
                "shard_off": int(self.shard.start), "shard_len": int(self.shard_len), "zero_stage": int(self.zero_stage)}
        return tensors, meta

    def load_optimizer_state(self, tensors: dict, meta: dict) -> None:
        """Strict: the state must come from the same rank of a run with the same number of ranks and the same shard."""
        from ..core.errors import SerializationError
        want = {"world": self.world, "rank": self.rank, "shard_off": int(self.shard.start), "shard_len": int(self.shard_len),
                "zero_stage": int(self.zero_stage)}
        got = {k: int(meta.get(k, want[k] if k == "zero_stage" else -1)) for k in want}
        if got != want:
            raise SerializationError(f"optimizer state was saved for {got}, this rank is {want}")
        if self.comm is not None:
            m, v = self.comm.optimizer_shard()
        else:
            m, v = self.engine.params.m, self.engine.params.v
        for name, dst in (("adam.m", m), ("adam.v", v)):
            if name not in tensors or tuple(tensors[name].shape) != tuple(dst.shape):
                raise SerializationError(f"optimizer state: {name} missing or of the wrong size")
        m.copy_(tensors["adam.m"].to(m.device))
        v.copy_(tensors["adam.v"].to(v.device))
        self.engine.step_count = int(meta["step"])
