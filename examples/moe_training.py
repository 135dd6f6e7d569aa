"""Mixture-of-experts training: a token classifier whose feed-forward block is a top-2 routed expert layer; the load
balancing loss is added to the task loss and the routing statistics are printed before and after
(crates/nn/examples/moe_training.rs).  The inputs come from four clusters, so that experts can specialise.

    python examples/moe_training.py [--steps 200] [--experts 4] [--device cuda:0]
"""
import torch

from _common import backend_for, parser

from rustral_b200.core import ForwardCtx
from rustral_b200.core.module import Module, Trainable
from rustral_b200.nn import CrossEntropyLoss, ExpertLayer, LayerNorm, LinearBuilder, MoEConfig
from rustral_b200.optim import Adam


class MoEClassifier(Module, Trainable):
    def __init__(self, backend, d_model, experts, classes, seed):
        self.inp = LinearBuilder(8, d_model).with_bias().seed(seed).build(backend)
        self.norm = LayerNorm.new(backend, d_model)
        self.moe = ExpertLayer.new(backend, MoEConfig(d_model, experts, 2 * d_model, top_k=2, capacity_factor=1.5), seed + 1)
        self.head = LinearBuilder(d_model, classes).with_bias().seed(seed + 2).build(backend)

    def forward(self, x, ctx):
        h = self.inp(x, ctx)
        out = self.moe(self.norm(h, ctx), ctx)
        return self.head((h + out.output).contiguous(), ctx), out.aux_loss


def clusters(n, seed):
    g = torch.Generator().manual_seed(seed)
    centres = torch.randn(4, 8, generator=g) * 2.0
    y = torch.randint(0, 4, (n,), generator=g)
    return centres[y] + 0.5 * torch.randn(n, 8, generator=g), y


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--experts", type=int, default=4)
    a = ap.parse_args(argv)
    backend = backend_for(a.device)
    dev, dt = backend.device(), backend.dtype
    x, y = clusters(2048, a.seed)
    x, y = x.to(dev, dt), y.to(dev)
    net, opt, ce = MoEClassifier(backend, 64, a.experts, 4, a.seed), Adam(lr=3e-3), CrossEntropyLoss()

    def routing():
        with torch.no_grad():
            ctx = ForwardCtx.inference()
            return net.moe.stats(net.norm(net.inp(x[:512], ctx), ctx))
    st0 = routing()
    print(f"before: tokens per expert {st0.tokens_per_expert}, imbalance {st0.load_imbalance:.2f}, dropped {st0.dropped_tokens}")
    g = torch.Generator().manual_seed(a.seed + 1)
    for step in range(a.steps):
        idx = torch.randint(0, len(x), (128,), generator=g).to(dev)
        net.zero_grad()
        logits, aux = net.forward(x[idx], ForwardCtx.train(backend))
        task = ce(logits.float(), y[idx])
        (task + aux).backward()
        opt.step(net.parameters())
        if step % 50 == 0 or step == a.steps - 1:
            print(f"step {step}: task loss {float(task.detach()):.4f}  balance loss {float(aux.detach()):.5f}")
    st1 = routing()
    with torch.no_grad():
        acc = float((net.forward(x, ForwardCtx.inference())[0].float().argmax(-1) == y).float().mean())
    print(f"after:  tokens per expert {st1.tokens_per_expert}, imbalance {st1.load_imbalance:.2f}, dropped {st1.dropped_tokens}; accuracy {acc:.3f}")
    return {"accuracy": acc, "imbalance_before": st0.load_imbalance, "imbalance_after": st1.load_imbalance,
            "tokens_per_expert": st1.tokens_per_expert}


if __name__ == "__main__":
    main()
