"""A small residual network for image classification: stem convolution, residual blocks (conv - BatchNorm - ReLU - conv -
BatchNorm, plus the skip), global max pooling and a linear head (crates/nn/examples/resnet_image_classification.rs).
Trained on generated seven-segment digit images.

    python examples/resnet_image_classification.py [--epochs 4] [--blocks 2] [--device cuda:0]
"""
import torch

from _common import backend_for, parser
from _synthetic import digit_images

from rustral_b200.core import ForwardCtx
from rustral_b200.core.module import Module, Trainable
from rustral_b200.nn import BatchNorm, Conv2d, Conv2dConfig, CrossEntropyLoss, LinearBuilder, global_max_pool2d, max_pool2d
from rustral_b200.optim import AdamW, WarmupCosine


class ResidualBlock(Module, Trainable):
    def __init__(self, backend, channels, seed):
        self.conv1 = Conv2d.new(backend, Conv2dConfig(channels, 3, 3, bias=False, in_channels=channels), seed=seed)
        self.bn1 = BatchNorm.new(backend, channels)
        self.conv2 = Conv2d.new(backend, Conv2dConfig(channels, 3, 3, bias=False, in_channels=channels), seed=seed + 1)
        self.bn2 = BatchNorm.new(backend, channels)

    def forward(self, x, ctx):
        h = torch.relu(self.bn1(self.conv1(x, ctx), ctx))
        return torch.relu(x + self.bn2(self.conv2(h, ctx), ctx))


class SmallResNet(Module, Trainable):
    def __init__(self, backend, channels=16, blocks=2, classes=10, seed=0):
        self.stem = Conv2d.new(backend, Conv2dConfig(channels, 3, 3, in_channels=1), seed=seed)
        self.blocks = [ResidualBlock(backend, channels, seed + 10 * (i + 1)) for i in range(blocks)]
        self.head = LinearBuilder(channels, classes).with_bias().seed(seed + 5).build(backend)

    def forward(self, x, ctx):
        x = max_pool2d(torch.relu(self.stem(x, ctx)), 2)
        for b in self.blocks:
            x = b.forward(x, ctx)
        return self.head(global_max_pool2d(x).contiguous(), ctx)


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--epochs", type=int, default=4)
    ap.add_argument("--blocks", type=int, default=2)
    ap.add_argument("--train", type=int, default=768)
    ap.add_argument("--batch", type=int, default=64)
    a = ap.parse_args(argv)
    backend = backend_for(a.device)
    dev, dt = backend.device(), backend.dtype
    xtr, ytr = digit_images(a.train, seed=a.seed)
    xte, yte = digit_images(256, seed=a.seed + 1)
    xtr, xte, ytr, yte = xtr.to(dev, dt), xte.to(dev, dt), ytr.to(dev), yte.to(dev)
    net = SmallResNet(backend, blocks=a.blocks, seed=a.seed)
    steps = a.epochs * ((a.train + a.batch - 1) // a.batch)
    opt = AdamW(lr=1e-2, weight_decay=1e-4)
    sched = WarmupCosine(1e-2, 1e-4, max(1, steps // 10), steps).attach(opt)
    loss_fn = CrossEntropyLoss()
    names = [n for n, _ in net.named_parameters()]
    print(f"{net.num_parameters()} parameters in {len(names)} tensors, e.g. {names[0]}, {names[3]}")
    for epoch in range(a.epochs):
        perm = torch.randperm(a.train, generator=torch.Generator().manual_seed(a.seed + epoch)).to(dev)
        total = 0.0
        for i in range(0, a.train, a.batch):
            idx = perm[i:i + a.batch]
            net.zero_grad()
            loss = loss_fn(net.forward(xtr[idx], ForwardCtx.train(backend)).float(), ytr[idx])
            loss.backward()
            opt.step(net.parameters())
            sched.step()
            total += float(loss.detach()) * len(idx)
        with torch.no_grad():
            acc = float((net.forward(xte, ForwardCtx.inference()).float().argmax(-1) == yte).float().mean())
        print(f"epoch {epoch}: loss {total / a.train:.4f}  lr {opt.lr:.2e}  test accuracy (running statistics) {acc:.3f}")
    return {"accuracy": acc, "parameters": net.num_parameters(), "names": names}


if __name__ == "__main__":
    main()
