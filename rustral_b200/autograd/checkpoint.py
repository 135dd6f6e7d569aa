"""Activation checkpointing with real recomputation (crates/autodiff/src/checkpoint.rs:29-300).

`checkpoint_segment(fn, *inputs)` runs `fn` without keeping its intermediate activations and re-runs it during
the backward pass; the reference's function of that name runs the forward normally and never recomputes
(checkpoint.rs:99-129)."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class CheckpointConfig:
    enabled: bool = True
    checkpoint_every_n_layers: int = 2
    preserve_patterns: list = field(default_factory=list)

    def should_checkpoint(self, layer_idx: int) -> bool:
        return self.enabled and self.checkpoint_every_n_layers > 0 and layer_idx % self.checkpoint_every_n_layers == 1


class _CheckpointFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, n_inputs, *args):
        ctx.fn = fn
        inputs, params = args[:n_inputs], args[n_inputs:]
        ctx.save_for_backward(*[a for a in args if isinstance(a, torch.Tensor)])
        ctx.is_tensor = [isinstance(a, torch.Tensor) for a in args]
        ctx.non_tensors = [a for a in args if not isinstance(a, torch.Tensor)]
        ctx.n_inputs = n_inputs
        with torch.no_grad():
            return fn(*inputs)

    @staticmethod
    def backward(ctx, *grad_out):
        saved = list(ctx.saved_tensors)
        nts = list(ctx.non_tensors)
        args = [saved.pop(0) if is_t else nts.pop(0) for is_t in ctx.is_tensor]
        detached = [a.detach().requires_grad_(a.requires_grad) if isinstance(a, torch.Tensor) and a.is_floating_point() else a
                    for a in args[:ctx.n_inputs]]
        params = args[ctx.n_inputs:]
        with torch.enable_grad():
            out = ctx.fn(*detached)
        outs = out if isinstance(out, tuple) else (out,)
        wrt = [a for a in detached if isinstance(a, torch.Tensor) and a.requires_grad] + [p for p in params if p.requires_grad]
        grads = torch.autograd.grad(outs, wrt, grad_out, allow_unused=True)
        it = iter(grads)
        res = []
        for a in detached:
            res.append(next(it) if isinstance(a, torch.Tensor) and a.requires_grad else None)
        for p in params:
            res.append(next(it) if p.requires_grad else None)
        return (None, None, *res)


class CheckpointedSegment:
    """A segment of the forward pass kept as (input, function) instead of its activations
    (crates/autodiff/src/checkpoint.rs:64-93): `recompute(ctx)` runs the function on the saved input again, which is what
    the backward pass of `checkpoint_segment` does internally.  `input_id` / `output_id` are the tape ids when the
    segment was recorded on a tape, else None."""

    def __init__(self, input_value: torch.Tensor, forward_fn, input_id=None, output_id=None):
        self.input_value = input_value.detach()
        self.forward_fn = forward_fn
        self.input_id, self.output_id = input_id, output_id

    def recompute(self, ctx=None) -> torch.Tensor:
        return self.forward_fn(self.input_value, ctx) if ctx is not None else self.forward_fn(self.input_value)

    def saved_bytes(self) -> int:
        return self.input_value.numel() * self.input_value.element_size()


def checkpoint_segment(fn, *inputs, parameters=()):
    """Runs `fn(*inputs)` keeping only `inputs`; activations inside are recomputed in the backward pass.  Parameters used
    inside `fn` must be listed in `parameters` (their tensors) so that they receive gradients."""
    return _CheckpointFn.apply(fn, len(inputs), *inputs, *parameters)


class CheckpointedTransformerLayer:
    """Wraps a layer `layer(x, ctx)`; layers whose index satisfies the config are recomputed in backward."""

    def __init__(self, layer, layer_idx: int, config: CheckpointConfig):
        self.layer, self.layer_idx, self.config = layer, layer_idx, config

    def __call__(self, x, ctx):
        if not self.config.should_checkpoint(self.layer_idx) or not torch.is_grad_enabled():
            return self.layer(x, ctx)
        params = [p.tensor for p in self.layer.parameters()]
        return checkpoint_segment(lambda t: self.layer(t, ctx), x, parameters=params)

    def parameters(self):
        return self.layer.parameters()

    def named_parameters(self):
        return self.layer.named_parameters()


class CheckpointManager:
    def __init__(self, config: CheckpointConfig | None = None):
        self.config = config or CheckpointConfig()
        self.recomputed = 0

    def wrap(self, layers: list) -> list:
        return [CheckpointedTransformerLayer(l, i, self.config) for i, l in enumerate(layers)]


@dataclass
class MemoryStats:
    """Analytic activation memory of a transformer stack with and without checkpointing."""
    without_bytes: int
    with_bytes: int

    @classmethod
    def calculate(cls, num_layers: int, batch: int, seq: int, d_model: int, ffn_dim: int, every_n: int = 2, elem_bytes: int = 2):
        per_layer = batch * seq * (8 * d_model + 2 * ffn_dim) * elem_bytes
        boundary = batch * seq * d_model * elem_bytes
        ck = num_layers // max(1, every_n)
        return cls(num_layers * per_layer, (num_layers - ck) * per_layer + ck * boundary + per_layer)

    @property
    def savings(self) -> float:
        return 1.0 - self.with_bytes / max(1, self.without_bytes)


def checkpoint_model(layers: list, config: CheckpointConfig | None = None) -> list:
    return CheckpointManager(config).wrap(layers)
