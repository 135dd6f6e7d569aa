"""XOR with a two-layer perceptron, twice: a hand-written loop over the tape, then the `Trainer` builder
(crates/nn/examples/xor.rs, crates/runtime/examples/tape_xor_classification.rs, crates/autodiff/examples/train_demo.rs).

    python examples/xor.py [--epochs 400] [--device cuda:0]
"""
import torch

from _common import backend_for, parser

from rustral_b200.autograd.tape import Tape
from rustral_b200.core import ForwardCtx
from rustral_b200.core.module import Module, Trainable
from rustral_b200.nn import LinearBuilder
from rustral_b200.optim import Adam
from rustral_b200.runtime.tape_trainer import SupervisedTapeModel, Trainer

DATA = [([0.0, 0.0], 0), ([0.0, 1.0], 1), ([1.0, 0.0], 1), ([1.0, 1.0], 0)]


class XorNet(Module, Trainable, SupervisedTapeModel):
    def __init__(self, backend, hidden=8, seed=0):
        self.l1 = LinearBuilder(2, hidden).with_bias().seed(seed).build(backend)
        self.l2 = LinearBuilder(hidden, 2).with_bias().seed(seed + 1).build(backend)
        self._device, self._dtype = backend.device(), backend.dtype

    def forward_tape(self, x, tape, ctx):
        xi = tape.constant(x)
        w1, b1 = tape.watch_parameter(self.l1.weight), tape.watch_parameter(self.l1.bias)
        w2, b2 = tape.watch_parameter(self.l2.weight), tape.watch_parameter(self.l2.bias)
        h = tape.tanh(tape.linear_tape(xi, w1, b1))
        return tape.linear_tape(h, w2, b2)

    def collate(self, xs):
        return torch.tensor(xs, dtype=self._dtype, device=self._device)

    def collate_targets(self, ys):
        return torch.tensor(ys, dtype=torch.int64, device=self._device)

    def predict(self, xs):
        ctx = ForwardCtx.inference()
        tape = Tape(ctx)
        return tape.value(self.forward_tape(self.collate(xs), tape, ctx)).float().argmax(-1).tolist()


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--epochs", type=int, default=400)
    a = ap.parse_args(argv)
    backend = backend_for(a.device)

    # 1. the loop written out: tape -> loss -> backward -> gradients by parameter -> optimizer
    net, opt = XorNet(backend, seed=a.seed), Adam(lr=0.05)
    xs, ys = net.collate([x for x, _ in DATA]), net.collate_targets([y for _, y in DATA])
    first = last = None
    for step in range(a.epochs):
        ctx = ForwardCtx.train(backend)
        tape = Tape(ctx)
        loss = tape.cross_entropy_loss(net.forward_tape(xs, tape, ctx), ys)
        grads = tape.backward(loss)
        opt.step(net.parameters(), {p.id: grads.param_gradient(p) for p in net.parameters()})
        last = float(tape.value(loss).detach())
        first = last if first is None else first
    manual = net.predict([x for x, _ in DATA])
    print(f"manual loop: loss {first:.4f} -> {last:.4f}, predictions {manual}")

    # 2. the same model through the trainer builder
    net2 = XorNet(backend, seed=a.seed)
    report = Trainer.classification(Adam(lr=0.05)).epochs(a.epochs).batch_size(4).shuffle(True).seed(a.seed).fit(backend, net2, DATA)
    built = net2.predict([x for x, _ in DATA])
    print(f"trainer: final loss {report.epochs[-1].mean_loss:.4f}, accuracy {report.accuracy:.2f}, predictions {built}")
    return {"manual": manual, "trainer": built, "loss_first": first, "loss_last": last, "accuracy": report.accuracy}


if __name__ == "__main__":
    main()
