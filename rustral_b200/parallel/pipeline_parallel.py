"""Pipeline parallelism: stage splitting and GPipe / 1F1B schedules over point-to-point sends
(crates/distributed/src/pipeline_parallel.rs:43-416).

Each rank owns one stage.  Activations travel forward and gradients backward through ProcessGroup.send / recv
(NCCL p2p on GPUs, on a side stream so transfers overlap the compute of the next micro-batch; gloo or the
threaded group on CPU).  Both schedules run real backward passes and return real losses; the reference's
schedules push literal 0.0 losses and never run backward (pipeline_parallel.rs:284-333).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch

from .process_group import DistributedError, ProcessGroup


class PipelineSchedule(enum.Enum):
    SIMPLE = "gpipe"             # all forwards, then all backwards
    INTERLEAVED = "1f1b"         # warm-up, steady one-forward-one-backward, cool-down
    ZERO_BUBBLE = "zero_bubble"  # 1F1B order with weight-gradient work deferred to fill the bubble


@dataclass
class PipelineConfig:
    num_micro_batches: int = 4
    schedule: PipelineSchedule = PipelineSchedule.INTERLEAVED
    checkpoint_activations: bool = False
    async_comm: bool = True


class StageSplitter:
    @staticmethod
    def split_by_count(num_layers: int, num_stages: int) -> list:
        """Contiguous ranges whose sizes differ by at most one, the larger ones first.  (The reference gives every stage
        ceil(L / S) layers, pipeline_parallel.rs:163-179, which leaves the last stage empty for 5 layers on 4 stages; an
        idle stage is an idle GPU.  The two rules agree whenever S divides L.)"""
        if num_stages <= 0:
            raise DistributedError("num_stages must be positive")
        base, extra = divmod(num_layers, num_stages)
        out, start = [], 0
        for s in range(num_stages):
            n = base + (1 if s < extra else 0)
            out.append(list(range(start, start + n)))
            start += n
        return out

    @staticmethod
    def balance_by_params(param_counts: list, num_stages: int) -> list:
        """Greedy contiguous split aiming at total / S parameters per stage (pipeline_parallel.rs:182-209)."""
        total = sum(param_counts)
        target = total / num_stages
        stages, cur, acc = [], [], 0.0
        remaining_stages = num_stages
        for i, n in enumerate(param_counts):
            layers_left = len(param_counts) - i
            # cut when the stage is full, or when every layer that is left is needed to give the later stages one each
            full = acc + n / 2 > target and layers_left >= remaining_stages - 1
            if cur and remaining_stages > 1 and (full or layers_left == remaining_stages - 1):
                stages.append(cur)
                remaining_stages -= 1
                cur, acc = [], 0.0
            cur.append(i)
            acc += n
        stages.append(cur)
        while len(stages) < num_stages:
            stages.append([])
        return stages

    auto_split = split_by_count


def pipeline_bubble_fraction(schedule: PipelineSchedule, num_stages: int, num_micro: int) -> float:
    """Idle share of a stage's time, with forward, input-gradient and weight-gradient passes of equal length t (so one
    micro-batch costs 3t).  GPipe and 1F1B idle for (S - 1) whole micro-batches: (S - 1) / (M + S - 1).  The zero-bubble
    schedule sends the input gradient on before it does the weight-gradient work, which shortens the wait of each
    earlier stage from t_F + t_B + t_W to t_F + t_B - t_W per hop: (S - 1) / (3 M + S - 1)."""
    if schedule is PipelineSchedule.ZERO_BUBBLE:
        return (num_stages - 1) / (3 * num_micro + num_stages - 1)
    return (num_stages - 1) / (num_micro + num_stages - 1)


class PipelineStage:
    """One stage: `forward_fn(x) -> y` built from this rank's layers, differentiable with torch.autograd."""

    def __init__(self, stage_id: int, num_stages: int, forward_fn, parameters):
        self.stage_id, self.num_stages = stage_id, num_stages
        self.forward_fn = forward_fn
        self.parameters = list(parameters)

    @property
    def is_first(self):
        return self.stage_id == 0

    @property
    def is_last(self):
        return self.stage_id == self.num_stages - 1


class PipelineParallel:
    """Runs one training step over `num_micro_batches` micro-batches.

    first stage:  micro-batch inputs come from `inputs[i]`
    last stage:   `loss_fn(output, targets[i]) -> scalar`
    other stages: activation shape / dtype come from `act_shape`, `act_dtype`.
    """

    def __init__(self, stage: PipelineStage, process_group: ProcessGroup, config: PipelineConfig, act_shape, act_dtype=torch.float32,
                 device="cpu"):
        if process_group.world_size != stage.num_stages:
            raise DistributedError("one rank per pipeline stage is required")
        self.stage, self.pg, self.cfg = stage, process_group, config
        self.act_shape, self.act_dtype, self.device = tuple(act_shape), act_dtype, torch.device(device)
        self._comm_stream = torch.cuda.Stream(self.device) if (self.device.type == "cuda" and config.async_comm) else None
        self.after_backward = None      # optional callable run after every micro-batch backward (e.g. fp32 accumulation)
        self.deferred_weight_grads = 0  # weight-gradient jobs that ran after their input gradient had been sent on

    # ---- p2p ------------------------------------------------------------------------------------------------------------
    def _recv(self, src: int, tag: int) -> torch.Tensor:
        buf = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
        if self._comm_stream is not None:
            with torch.cuda.stream(self._comm_stream):
                self.pg.recv(buf, src, tag)
            torch.cuda.current_stream().wait_stream(self._comm_stream)
        else:
            self.pg.recv(buf, src, tag)
        return buf

    def _send(self, t: torch.Tensor, dst: int, tag: int) -> None:
        if self._comm_stream is not None:
            self._comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._comm_stream):
                self.pg.send(t, dst, tag)
            t.record_stream(self._comm_stream)
        else:
            self.pg.send(t, dst, tag)

    # ---- one micro-batch forward / backward -----------------------------------------------------------------------------
    def _forward(self, i: int, inputs, targets, loss_fn, saved: dict, losses: list) -> None:
        st = self.stage
        if st.is_first:
            x = inputs[i]
        else:
            x = self._recv(st.stage_id - 1, 2 * i).requires_grad_(True)
        y = st.forward_fn(x)
        if st.is_last:
            loss = loss_fn(y, targets[i]) / self.cfg.num_micro_batches
            losses.append(loss.detach())
            saved[i] = (x, loss)
        else:
            self._send(y.detach(), st.stage_id + 1, 2 * i)
            saved[i] = (x, y)

    def _backward(self, i: int, saved: dict) -> None:
        st = self.stage
        x, out = saved.pop(i)
        g = None if st.is_last else self._recv(st.stage_id + 1, 2 * i + 1)
        if self.cfg.schedule is PipelineSchedule.ZERO_BUBBLE:
            # input gradients first; the previous stage gets its gradient before this stage starts on the weight
            # gradients of its linear layers, which then run while that stage already works on its own backward pass
            from ..ops.matmul import WeightGradStore
            with WeightGradStore.defer() as deferred:
                out.backward(g)
            if not st.is_first:
                self._send(x.grad, st.stage_id - 1, 2 * i + 1)
            self.deferred_weight_grads += len(deferred)
            WeightGradStore.run(deferred)
        else:
            out.backward(g)
            if not st.is_first:
                self._send(x.grad, st.stage_id - 1, 2 * i + 1)
        if self.after_backward is not None:
            self.after_backward()

    def train_step(self, inputs=None, targets=None, loss_fn=None) -> torch.Tensor | None:
        """Gradients accumulate in the stage's parameters (zero them beforehand).  Returns the mean loss on the last
        stage, None elsewhere."""
        M, S, s = self.cfg.num_micro_batches, self.stage.num_stages, self.stage.stage_id
        saved, losses = {}, []
        if self.cfg.schedule is PipelineSchedule.SIMPLE:
            for i in range(M):
                self._forward(i, inputs, targets, loss_fn, saved, losses)
            for i in range(M):
                self._backward(i, saved)
        else:
            warm = min(M, S - 1 - s)
            f = b = 0
            for _ in range(warm):
                self._forward(f, inputs, targets, loss_fn, saved, losses)
                f += 1
            while f < M:                       # steady state: one forward, one backward
                self._forward(f, inputs, targets, loss_fn, saved, losses)
                f += 1
                self._backward(b, saved)
                b += 1
            while b < M:                       # cool-down
                self._backward(b, saved)
                b += 1
        if self._comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self._comm_stream)
        return torch.stack(losses).sum() if losses else None

    def pipeline_stats(self) -> "PipelineStats":
        bubble = pipeline_bubble_fraction(self.cfg.schedule, self.stage.num_stages, self.cfg.num_micro_batches)
        return PipelineStats(self.stage.num_stages, self.cfg.num_micro_batches, self.cfg.schedule.name, bubble, 1.0 - bubble)


@dataclass
class PipelineStats:
    """crates/distributed/src/pipeline_parallel.rs:339-375.  Also answers the dictionary keys of the same names."""
    num_stages: int
    num_micro_batches: int
    schedule: str
    bubble_fraction: float
    efficiency: float

    def __getitem__(self, key):
        return getattr(self, key)


class PipelineLayer:
    """What a pipeline stage accepts as a layer: a module with `forward(x, ctx)` and `parameters()` (the reference's blanket
    trait, pipeline_parallel.rs:109-111).  `PipelineLayer.check(obj)` says whether an object qualifies."""

    @staticmethod
    def check(obj) -> bool:
        return callable(getattr(obj, "forward", None)) and callable(getattr(obj, "parameters", None))


class PipelineComm:
    """Point-to-point channel between adjacent stages (crates/distributed/src/pipeline_parallel.rs:377-413, where the
    queues are in-process `Mutex<Vec>`s).  Tags keep activations (even) and gradients (odd) of a micro-batch apart."""

    def __init__(self, process_group: ProcessGroup, stage_id: int, num_stages: int):
        self.pg, self.stage_id, self.num_stages = process_group, stage_id, num_stages

    def send_activation(self, t: torch.Tensor, micro_batch: int) -> None:
        if self.stage_id + 1 >= self.num_stages:
            raise DistributedError("the last stage has no successor")
        self.pg.send(t, self.stage_id + 1, 2 * micro_batch)

    def recv_activation(self, buf: torch.Tensor, micro_batch: int) -> torch.Tensor:
        if self.stage_id == 0:
            raise DistributedError("the first stage has no predecessor")
        return self.pg.recv(buf, self.stage_id - 1, 2 * micro_batch)

    def send_gradient(self, t: torch.Tensor, micro_batch: int) -> None:
        if self.stage_id == 0:
            raise DistributedError("the first stage has no predecessor")
        self.pg.send(t, self.stage_id - 1, 2 * micro_batch + 1)

    def recv_gradient(self, buf: torch.Tensor, micro_batch: int) -> torch.Tensor:
        if self.stage_id + 1 >= self.num_stages:
            raise DistributedError("the last stage has no successor")
        return self.pg.recv(buf, self.stage_id + 1, 2 * micro_batch + 1)


def create_pipeline(layers: list, process_group: ProcessGroup, config: PipelineConfig, act_shape, act_dtype=torch.float32,
                    device="cpu", ctx=None) -> PipelineParallel:
    """Splits `layers` (modules with forward(x, ctx)) evenly over the ranks of `process_group`."""
    S, r = process_group.world_size, process_group.rank
    mine = [layers[i] for i in StageSplitter.split_by_count(len(layers), S)[r]]

    def fwd(x):
        for l in mine:
            x = l(x, ctx) if ctx is not None else l(x)
        return x

    params = [p for l in mine for p in (l.parameters() if hasattr(l, "parameters") else [])]
    return PipelineParallel(PipelineStage(r, S, fwd, params), process_group, config, act_shape, act_dtype, device)


class SequentialStage:
    """A list of layers run in order: the stage type of the in-process `PipelineParallelTrainer`
    (crates/distributed/src/tensor_parallel.rs:192-236)."""

    def __init__(self, stage_id: int, num_stages: int, micro_batch_size: int):
        self.stage_id, self.num_stages, self.micro_batch_size = stage_id, num_stages, micro_batch_size
        self.layers: list = []

    def add_layer(self, layer) -> None:
        self.layers.append(layer)

    def forward(self, x, ctx=None):
        for layer in self.layers:
            x = layer(x, ctx)
        return x

    def parameters(self) -> list:
        return [p for l in self.layers if hasattr(l, "parameters") for p in l.parameters()]


class PipelineParallelTrainer:
    """All stages in ONE process, micro-batched (crates/distributed/src/tensor_parallel.rs:242-308): the batch is cut
    into micro-batches of the first stage's size, every micro-batch runs through all stages, the losses are averaged
    and (unlike the reference, whose backward returns its argument) gradients flow through torch.autograd and are
    accumulated over the micro-batches, so one optimizer step follows the call.  The multi-rank pipeline is
    `PipelineParallel`."""

    def __init__(self, num_stages: int):
        self.num_stages = num_stages
        self.stages: list = []

    def add_stage(self, stage: SequentialStage) -> None:
        if len(self.stages) >= self.num_stages:
            raise DistributedError("more stages than num_stages")
        self.stages.append(stage)

    def forward(self, x, ctx=None):
        for st in self.stages:
            x = st.forward(x, ctx)
        return x

    def parameters(self) -> list:
        return [p for st in self.stages for p in st.parameters()]

    def split_into_micro_batches(self, batch) -> list:
        mb = self.stages[0].micro_batch_size if self.stages else 1
        return [batch[i:i + mb] for i in range(0, len(batch), mb)]

    def train_step(self, batch, loss_fn, ctx=None) -> float:
        """`loss_fn(micro_batch, forward, ctx) -> scalar loss tensor`, where `forward` is this trainer's forward.
        Returns the mean micro-batch loss; parameter `.grad`s hold the gradient of that mean."""
        micro = self.split_into_micro_batches(batch)
        if not micro:
            return 0.0
        total = 0.0
        for mb in micro:
            loss = loss_fn(mb, self.forward, ctx)
            (loss / len(micro)).backward()
            total += float(loss.detach())
        return total / len(micro)
