"""3-D parallel training: data x pipeline x tensor over a DeviceMesh (crates/distributed/src/parallelism_3d.rs:35-333).

The trainer owns this rank's pipeline stage (whose layers may be tensor-parallel), runs the 1F1B schedule over
the pipeline group, then averages gradients over the data-parallel group and steps the optimizer.  In the reference
the step is placeholders (loss 0.0, no-op reductions, parallelism_3d.rs:98-192)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .data_parallel import all_reduce_gradients
from .device_mesh import DeviceMesh
from .pipeline_parallel import PipelineConfig, PipelineParallel, PipelineSchedule, PipelineStage
from .process_group import DistributedError, ProcessGroup


@dataclass
class Parallel3DConfig:
    dp: int = 1
    tp: int = 1
    pp: int = 1
    gradient_accumulation_steps: int = 1
    pipeline_num_microbatches: int = 4

    def validate(self, world_size: int) -> None:
        if self.dp * self.tp * self.pp != world_size:
            raise DistributedError(f"dp*tp*pp = {self.dp * self.tp * self.pp} != world size {world_size}")

    def total_gpus(self) -> int:
        return self.dp * self.tp * self.pp


class Parallel3DTrainer:
    def __init__(self, mesh: DeviceMesh, stage: PipelineStage, optimizer, dp_group: ProcessGroup, pp_group: ProcessGroup,
                 tp_group: ProcessGroup | None, config: Parallel3DConfig, act_shape, act_dtype=torch.float32, device="cpu"):
        self.mesh, self.stage, self.optimizer = mesh, stage, optimizer
        self.dp_group, self.pp_group, self.tp_group, self.config = dp_group, pp_group, tp_group, config
        self.pipeline = PipelineParallel(stage, pp_group, PipelineConfig(config.pipeline_num_microbatches,
                                                                        PipelineSchedule.INTERLEAVED), act_shape, act_dtype, device)

    def scatter_batch(self, batch: torch.Tensor) -> torch.Tensor:
        """This data-parallel rank's contiguous slice of dim 0."""
        per = batch.shape[0] // self.dp_group.world_size
        return batch[self.dp_group.rank * per:(self.dp_group.rank + 1) * per]

    def step(self, inputs=None, targets=None, loss_fn=None):
        """inputs / targets: lists of micro-batches for this data-parallel rank (first / last stage only)."""
        for p in self.stage.parameters:
            p.zero_grad()
        loss = self.pipeline.train_step(inputs, targets, loss_fn)
        grads = [p.tensor.grad for p in self.stage.parameters if p.tensor.grad is not None]
        all_reduce_gradients(self.dp_group, grads, average=True)
        self.optimizer.step(self.stage.parameters)
        if loss is not None:
            l = loss.detach().float().reshape(1).clone()
            self.dp_group.all_reduce_mean(l, "loss3d")
            return float(l)
        return None


class Parallel3DLayer:
    """One tensor-parallel linear layer inside a 3-D parallel model: column-parallel over the mesh's tensor group
    (crates/distributed/src/parallelism_3d.rs:216-243).  `gather_output=False` keeps the output sharded for a
    following row-parallel layer."""

    def __init__(self, in_features: int, out_features: int, tp_group: ProcessGroup, backend, gather_output: bool = True,
                 bias: bool = False, seed: int = 42):
        from .tensor_parallel import TensorParallelLinear
        self.tp_group = tp_group
        self.linear = TensorParallelLinear.column_parallel(backend, in_features, out_features, tp_group, bias=bias, seed=seed,
                                                           gather_output=gather_output)

    def forward(self, x, ctx=None):
        return self.linear(x, ctx)

    __call__ = forward

    def parameters(self) -> list:
        return self.linear.parameters()

    def named_parameters(self) -> list:
        return [("linear." + n, p) for n, p in self.linear.named_parameters()]


def create_3d_parallel_model(build_layer, num_layers: int, mesh: DeviceMesh) -> list:
    """This rank's layers: the contiguous slice of `num_layers` owned by its pipeline coordinate; `build_layer(i)`
    constructs layer i (tensor-parallel inside, if it wants, from the mesh's tp group)."""
    pp = mesh.shape[mesh.dim_names.index("pp")]
    me = mesh.my_coord[mesh.dim_names.index("pp")]
    per = (num_layers + pp - 1) // pp
    return [build_layer(i) for i in range(me * per, min(num_layers, (me + 1) * per))]
