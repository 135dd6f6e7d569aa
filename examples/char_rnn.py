"""Character-level language model: embedding -> stacked LSTM -> linear head, trained with truncated back-propagation
through time on an embedded text, then sampled (crates/nn/examples/char_rnn.rs).

    python examples/char_rnn.py [--steps 150] [--hidden 96] [--layers 2] [--device cuda:0]
"""
import math

import torch

from _common import backend_for, parser
from _synthetic import TEXT

from rustral_b200.core import ForwardCtx
from rustral_b200.core.module import Module, Trainable
from rustral_b200.nn import CrossEntropyLoss, Embedding, LinearBuilder, StackedLstm
from rustral_b200.optim import Adam


class CharRnn(Module, Trainable):
    def __init__(self, backend, vocab, dim, hidden, layers, seed):
        self.embed = Embedding.new(backend, vocab, dim, seed, scale=0.1)
        self.rnn = StackedLstm.new(backend, dim, hidden, layers, seed + 1)
        self.head = LinearBuilder(hidden, vocab).with_bias().seed(seed + 2).build(backend)

    def forward(self, ids, ctx, states=None):
        """ids [T, B] -> logits [T, B, vocab] and the final (h, c) of every layer."""
        out, states = self.rnn.forward_sequence(self.embed(ids, ctx), ctx, states)
        return self.head(out.contiguous(), ctx), states


def sample(net, stoi, itos, prime, n, temperature, seed):
    g = torch.Generator().manual_seed(seed)
    ctx = ForwardCtx.inference()
    dev = net.head.weight.tensor.device
    ids = torch.tensor([[stoi[c]] for c in prime], device=dev)
    with torch.no_grad():
        logits, states = net.forward(ids, ctx)
        out = list(prime)
        for _ in range(n):
            p = torch.softmax(logits[-1, 0].float().cpu() / temperature, -1)
            nxt = int(torch.multinomial(p, 1, generator=g))
            out.append(itos[nxt])
            logits, states = net.forward(torch.tensor([[nxt]], device=dev), ctx, states)
    return "".join(out)


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--steps", type=int, default=150)
    ap.add_argument("--seq", type=int, default=32)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--hidden", type=int, default=96)
    ap.add_argument("--layers", type=int, default=2)
    a = ap.parse_args(argv)
    backend = backend_for(a.device)
    dev = backend.device()
    chars = sorted(set(TEXT))
    stoi, itos = {c: i for i, c in enumerate(chars)}, chars
    data = torch.tensor([stoi[c] for c in TEXT], device=dev)
    net, opt, loss_fn = CharRnn(backend, len(chars), 32, a.hidden, a.layers, a.seed), Adam(lr=5e-3, max_grad_norm=1.0), CrossEntropyLoss()
    g = torch.Generator().manual_seed(a.seed)
    first = last = None
    for step in range(a.steps):
        starts = torch.randint(0, len(data) - a.seq - 1, (a.batch,), generator=g)
        x = torch.stack([data[s:s + a.seq] for s in starts.tolist()], 1)              # [T, B]
        y = torch.stack([data[s + 1:s + a.seq + 1] for s in starts.tolist()], 1)
        net.zero_grad()
        logits, _ = net.forward(x, ForwardCtx.train(backend))
        loss = loss_fn(logits.reshape(-1, len(chars)).float(), y.reshape(-1))
        loss.backward()
        opt.step(net.parameters())
        last = float(loss.detach())
        first = last if first is None else first
        if step % 50 == 0 or step == a.steps - 1:
            print(f"step {step}: loss {last:.3f} (uniform would be {math.log(len(chars)):.3f})")
    text = sample(net, stoi, itos, "the ", 80, 0.7, a.seed)
    print("sample:", text)
    return {"loss_first": first, "loss_last": last, "sample": text, "vocab": len(chars)}


if __name__ == "__main__":
    main()
