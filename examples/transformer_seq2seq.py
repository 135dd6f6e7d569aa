"""Sequence-to-sequence transformer (encoder + decoder with cross-attention) learning to reverse a token sequence, with
teacher forcing in training and greedy decoding at the end (crates/nn/examples/transformer_seq2seq.rs).

    python examples/transformer_seq2seq.py [--steps 500] [--device cuda:0]
"""
import torch

from _common import backend_for, parser

from rustral_b200.core import ForwardCtx
from rustral_b200.nn import CrossEntropyLoss, TransformerEncoderConfig, TransformerEncoderDecoder
from rustral_b200.optim import Adam, WarmupCosine

BOS, EOS, FIRST = 1, 2, 3


def batch(n, length, vocab, g):
    src = torch.randint(FIRST, vocab, (n, length), generator=g)
    rev = torch.flip(src, (1,))
    tgt_in = torch.cat([torch.full((n, 1), BOS), rev], 1)                 # <bos> y1 .. yL
    tgt_out = torch.cat([rev, torch.full((n, 1), EOS)], 1)                # y1 .. yL <eos>
    return src, tgt_in, tgt_out


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--length", type=int, default=6)
    ap.add_argument("--vocab", type=int, default=16)
    a = ap.parse_args(argv)
    backend = backend_for(a.device)
    dev = backend.device()
    cfg = TransformerEncoderConfig(d_model=64, num_heads=4, num_layers=2, ff_dim=128, dropout=0.0, max_seq_len=32)
    model = TransformerEncoderDecoder.new(backend, cfg, a.vocab, a.vocab, seed=a.seed)
    with torch.no_grad():                      # token embeddings start at N(0, 0.02); the position table has unit size
        for emb in (model.encoder.token_embedding, model.decoder.token_embedding):
            emb.embed.tensor.mul_(10.0)
    opt = Adam(lr=2e-3)
    sched = WarmupCosine(2e-3, 1e-4, 20, a.steps).attach(opt)
    ce = CrossEntropyLoss()
    g = torch.Generator().manual_seed(a.seed)
    for step in range(a.steps):
        src, tin, tout = (t.to(dev) for t in batch(64, a.length, a.vocab, g))
        model.zero_grad()
        logits = model.forward((src, tin), ForwardCtx.train(backend))
        loss = ce(logits.reshape(-1, a.vocab).float(), tout.reshape(-1))
        loss.backward()
        opt.step(model.parameters())
        sched.step()
        if step % 100 == 0 or step == a.steps - 1:
            print(f"step {step}: loss {float(loss.detach()):.4f}")
    src, _, tout = batch(32, a.length, a.vocab, g)
    ctx = ForwardCtx.inference()
    exact = 0
    for i in range(len(src)):
        out = model.generate(src[i:i + 1].to(dev), ctx, bos=BOS, eos=EOS, max_len=a.length + 2)
        exact += int(out[1:] == tout[i].tolist())
    print(f"source {src[0].tolist()} -> generated {out if len(src) == 1 else model.generate(src[:1].to(dev), ctx, bos=BOS, eos=EOS, max_len=a.length + 2)}")
    print(f"exact reversals by greedy decoding: {exact}/{len(src)}")
    return {"loss": float(loss.detach()), "exact": exact, "total": len(src)}


if __name__ == "__main__":
    main()
