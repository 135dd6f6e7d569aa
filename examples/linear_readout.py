"""Label heads over feature vectors: a single-label `Readout` over a label vocabulary, a multi-label `MultiReadout`
with one sigmoid head per label, and a `BinaryReadout`; each trained for a few steps and asked for predictions with
probabilities (crates/nn/examples/linear_readout.rs).

    python examples/linear_readout.py [--device cuda:0]
"""
import torch

from _common import backend_for, parser

from rustral_b200.core import ForwardCtx
from rustral_b200.nn import BCEWithLogitsLoss, BinaryReadout, CrossEntropyLoss, MultiReadout, Readout
from rustral_b200.optim import Adam
from rustral_b200.symbolic import Vocabulary


def main(argv=None):
    a = parser(__doc__).parse_args(argv)
    backend = backend_for(a.device)
    dev, dt = backend.device(), backend.dtype
    g = torch.Generator().manual_seed(a.seed)
    labels = Vocabulary.with_specials("<unk>", ["negative", "neutral", "positive"])
    centres = torch.randn(len(labels), 12, generator=g) * 2
    y = torch.randint(1, len(labels), (256,), generator=g)               # id 0 is <unk> and never a target
    x = (centres[y] + 0.3 * torch.randn(256, 12, generator=g)).to(dev, dt)

    single = Readout.new(backend, labels, 12, seed=a.seed)
    opt, ce = Adam(lr=0.05), CrossEntropyLoss()
    for _ in range(60):
        single.zero_grad()
        ce(single.logits(x, ForwardCtx.train(backend)).float(), y.to(dev)).backward()
        opt.step(single.parameters())
    preds = single.predict(x[:4], ForwardCtx.inference())
    for p, t in zip(preds, y[:4].tolist()):
        print(f"readout: {p.label:<9} p={p.score:.3f}   (truth: {labels.token(t)})")
    acc = sum(p.id == t for p, t in zip(single.predict(x, ForwardCtx.inference()), y.tolist())) / len(y)

    tags = ["urgent", "billing", "technical"]
    multi = MultiReadout.new(backend, tags, 12, seed=a.seed + 1)
    truth = (x[:, :3].float() > 0).float()                                  # tag j is on when feature j is positive
    opt, bce = Adam(lr=0.05), BCEWithLogitsLoss()
    for _ in range(80):
        multi.zero_grad()
        ctx = ForwardCtx.train(backend)
        logits = torch.cat([h(x, ctx) for h in multi.heads], -1).float()
        bce(logits, truth).backward()
        opt.step(multi.parameters())
    ctx = ForwardCtx.inference()
    first = multi.predict(x[:1], ctx)[0]
    print("multi-label:", [(p.label, round(p.score, 2)) for p in first], "top-2:", [(p.label, round(p.score, 2)) for p in multi.top_k(x[:1], ctx, 2)[0]])
    multi_acc = float(((multi.forward(x, ctx) >= 0.5).float().cpu() == truth.cpu()).float().mean())

    binary = BinaryReadout.new(backend, 12, seed=a.seed + 2)
    print("binary readout on 4 rows (untrained):", binary.predict(x[:4], ctx))
    print(f"accuracy: single-label {acc:.3f}, multi-label {multi_acc:.3f}")
    return {"accuracy": acc, "multi_accuracy": multi_acc, "first": [p.label for p in preds]}


if __name__ == "__main__":
    main()
