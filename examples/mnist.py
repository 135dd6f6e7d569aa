"""Digit classifier: two convolutions with max-pooling and a linear head, trained with Adam on procedurally drawn
seven-segment digits (crates/nn/examples/mnist.rs uses the same network shape on MNIST; this installation has no dataset
download, so the images are generated).

    python examples/mnist.py [--epochs 3] [--train 1024] [--device cuda:0]
"""
import torch

from _common import backend_for, parser
from _synthetic import digit_images

from rustral_b200.core import ForwardCtx
from rustral_b200.core.module import Module, Trainable
from rustral_b200.nn import Conv2d, Conv2dConfig, CrossEntropyLoss, LinearBuilder, max_pool2d
from rustral_b200.optim import Adam


class DigitNet(Module, Trainable):
    def __init__(self, backend, seed=0):
        self.c1 = Conv2d.new(backend, Conv2dConfig(8, 3, 3, in_channels=1), seed=seed)
        self.c2 = Conv2d.new(backend, Conv2dConfig(16, 3, 3, in_channels=8), seed=seed + 1)
        self.head = LinearBuilder(16 * 4 * 4, 10).with_bias().seed(seed + 2).build(backend)

    def forward(self, x, ctx):
        x = max_pool2d(torch.relu(self.c1(x, ctx)), 2)            # 16 -> 8
        x = max_pool2d(torch.relu(self.c2(x, ctx)), 2)            # 8 -> 4
        return self.head(x.reshape(x.shape[0], -1).contiguous(), ctx)


def accuracy(net, x, y):
    with torch.no_grad():
        return float((net.forward(x, ForwardCtx.inference()).float().argmax(-1) == y).float().mean())


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--epochs", type=int, default=6)
    ap.add_argument("--train", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=64)
    a = ap.parse_args(argv)
    backend = backend_for(a.device)
    dev, dt = backend.device(), backend.dtype
    xtr, ytr = digit_images(a.train, seed=a.seed)
    xte, yte = digit_images(256, seed=a.seed + 1)
    xtr, xte, ytr, yte = xtr.to(dev, dt), xte.to(dev, dt), ytr.to(dev), yte.to(dev)
    net, opt, loss_fn = DigitNet(backend, a.seed), Adam(lr=1e-2), CrossEntropyLoss()
    before = accuracy(net, xte, yte)
    for epoch in range(a.epochs):
        perm = torch.randperm(a.train, generator=torch.Generator().manual_seed(a.seed + epoch)).to(dev)
        total = 0.0
        for i in range(0, a.train, a.batch):
            idx = perm[i:i + a.batch]
            net.zero_grad()
            loss = loss_fn(net.forward(xtr[idx], ForwardCtx.train(backend)).float(), ytr[idx])
            loss.backward()
            opt.step(net.parameters())
            total += float(loss.detach()) * len(idx)
        print(f"epoch {epoch}: loss {total / a.train:.4f}  test accuracy {accuracy(net, xte, yte):.3f}")
    after = accuracy(net, xte, yte)
    return {"accuracy_before": before, "accuracy_after": after, "parameters": net.num_parameters()}


if __name__ == "__main__":
    main()
