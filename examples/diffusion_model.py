"""Denoising diffusion on a 2-D point cloud: an MLP predicts the noise added at a random timestep (sinusoidal time
embedding concatenated to the point), trained with the simple DDPM loss, then sampled by ancestral sampling
(crates/nn/examples/diffusion_model.rs).

    python examples/diffusion_model.py [--steps 600] [--timesteps 50] [--device cuda:0]
"""
import math

import torch

from _common import backend_for, parser
from _synthetic import two_moons

from rustral_b200.core import ForwardCtx
from rustral_b200.core.module import Module, Trainable
from rustral_b200.nn import LinearBuilder, MSELoss
from rustral_b200.optim import Adam


def time_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    freqs = torch.exp(torch.arange(dim // 2, device=t.device, dtype=torch.float32) * (-math.log(1000.0) / (dim // 2)))
    ang = t.float()[:, None] * freqs[None]
    return torch.cat([torch.sin(ang), torch.cos(ang)], 1)


class NoisePredictor(Module, Trainable):
    def __init__(self, backend, hidden=96, tdim=16, seed=0):
        self.tdim = tdim
        self.l1 = LinearBuilder(2 + tdim, hidden).with_bias().seed(seed).activation("gelu").build(backend)
        self.l2 = LinearBuilder(hidden, hidden).with_bias().seed(seed + 1).activation("gelu").build(backend)
        self.l3 = LinearBuilder(hidden, 2).with_bias().seed(seed + 2).build(backend)

    def forward(self, x, t, ctx):
        h = torch.cat([x, time_embedding(t, self.tdim).to(x.dtype)], 1).contiguous()
        return self.l3(self.l2(self.l1(h, ctx), ctx), ctx)


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--steps", type=int, default=600)
    ap.add_argument("--timesteps", type=int, default=50)
    ap.add_argument("--batch", type=int, default=256)
    a = ap.parse_args(argv)
    backend = backend_for(a.device)
    dev, dt = backend.device(), backend.dtype
    T = a.timesteps
    betas = torch.linspace(1e-4, 0.2, T, device=dev)
    alphas = 1.0 - betas
    abar = torch.cumprod(alphas, 0)
    data = (two_moons(4096, seed=a.seed) - torch.tensor([0.5, 0.25])).to(dev)
    net, opt, mse = NoisePredictor(backend, seed=a.seed), Adam(lr=2e-3), MSELoss()
    g = torch.Generator().manual_seed(a.seed)
    first = last = None
    for step in range(a.steps):
        idx = torch.randint(0, len(data), (a.batch,), generator=g).to(dev)
        t = torch.randint(0, T, (a.batch,), generator=g).to(dev)
        eps = torch.randn(a.batch, 2, generator=g).to(dev)
        x_t = abar[t].sqrt()[:, None] * data[idx] + (1 - abar[t]).sqrt()[:, None] * eps
        net.zero_grad()
        loss = mse(net.forward(x_t.to(dt), t, ForwardCtx.train(backend)).float(), eps)
        loss.backward()
        opt.step(net.parameters())
        last = float(loss.detach())
        first = last if first is None else first
        if step % 200 == 0 or step == a.steps - 1:
            print(f"step {step}: noise-prediction loss {last:.4f}")
    # ancestral sampling from pure noise
    with torch.no_grad():
        x = torch.randn(1024, 2, generator=g).to(dev)
        ctx = ForwardCtx.inference()
        for i in reversed(range(T)):
            t = torch.full((1024,), i, device=dev)
            eps_hat = net.forward(x.to(dt), t, ctx).float()
            x = (x - betas[i] / (1 - abar[i]).sqrt() * eps_hat) / alphas[i].sqrt()
            if i > 0:
                x = x + betas[i].sqrt() * torch.randn(1024, 2, generator=g).to(dev)
    # how close the samples are to the data: mean distance from a sample to its nearest data point
    near = torch.cdist(x, data[:1024]).min(1).values.mean()
    noise_near = torch.cdist(torch.randn(1024, 2, generator=g).to(dev), data[:1024]).min(1).values.mean()
    print(f"mean distance to the nearest data point: samples {float(near):.3f}, unit Gaussian noise {float(noise_near):.3f}")
    return {"loss_first": first, "loss_last": last, "sample_distance": float(near), "noise_distance": float(noise_near)}


if __name__ == "__main__":
    main()
