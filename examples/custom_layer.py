"""Writing a layer of your own: a gated residual unit built from `Parameter`s made by the backend, with named
parameters, gradient flow, parameter counting and a state-dict round trip coming from the module traits
(crates/core/examples/custom_layer.rs; saving to a file is crates/runtime/examples/save_linear_artifact.rs).

    python examples/custom_layer.py [--out artifact.safetensors] [--device cuda:0]
"""
import os
import tempfile

import torch

from _common import backend_for, parser

from rustral_b200.core import ForwardCtx
from rustral_b200.core.module import Module, Saveable, Trainable
from rustral_b200.nn import LayerNorm, LinearBuilder
from rustral_b200.optim import Sgd
from rustral_b200.runtime.model_io import load_model_from_path, save_model_to_path


class GatedResidual(Module, Trainable, Saveable):
    """y = x + sigmoid(x W_g^T + b_g) * (LayerNorm(x) W_v^T).  Attributes that are parameters, modules or lists of
    modules are found by the traits; nothing has to be registered."""

    def __init__(self, backend, dim, seed=0):
        self.norm = LayerNorm.new(backend, dim)
        self.value = LinearBuilder(dim, dim).seed(seed).build(backend)                    # a sub-module
        self.gate_weight = backend.normal_parameter("gate_weight", (dim, dim), seed + 1, dim ** -0.5)
        self.gate_bias = backend.constant_parameter("gate_bias", (dim,), -1.0)             # gates start mostly closed

    def forward(self, x, ctx):
        gate = torch.sigmoid(x @ self.gate_weight.tensor.t() + self.gate_bias.tensor)
        return x + gate * self.value(self.norm(x, ctx), ctx)


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    backend = backend_for(a.device)
    dev, dt = backend.device(), backend.dtype
    layer = GatedResidual(backend, 16, a.seed)
    names = [n for n, _ in layer.named_parameters()]
    print(f"{layer.num_parameters()} parameters:", ", ".join(names))
    x = torch.randn(8, 16, generator=torch.Generator().manual_seed(a.seed)).to(dev, dt)
    target = torch.roll(x, 1, dims=1)
    opt = Sgd(lr=0.1, momentum=0.9)
    losses = []
    for _ in range(50):
        layer.zero_grad()
        loss = (layer(x, ForwardCtx.train(backend)).float() - target.float()).square().mean()
        loss.backward()
        opt.step(layer.parameters())
        losses.append(float(loss.detach()))
    print(f"loss {losses[0]:.4f} -> {losses[-1]:.4f}; every parameter received a gradient: "
          f"{all(p.tensor.grad is not None for p in layer.parameters())}")
    path = a.out or os.path.join(tempfile.mkdtemp(), "gated_residual.safetensors")
    save_model_to_path(layer, path)
    copy = GatedResidual(backend, 16, a.seed + 100)
    load_model_from_path(copy, path)
    ctx = ForwardCtx.inference()
    same = torch.equal(layer(x, ctx), copy(x, ctx))
    print(f"wrote {os.path.getsize(path)} bytes to {path}; a fresh layer loaded from it gives identical outputs: {same}")
    return {"names": names, "loss_first": losses[0], "loss_last": losses[-1], "roundtrip": same, "path": path}


if __name__ == "__main__":
    main()
