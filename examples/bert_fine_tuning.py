"""BERT-style two-stage training on generated data: (1) masked-token pre-training of a bidirectional transformer encoder
on sequences drawn from two "topics" with their own token statistics, (2) fine-tuning a classification head on the first
position's representation with a smaller learning rate for the encoder than for the new head
(crates/nn/examples/bert_fine_tuning.rs, transformer_bert_encoder.rs).

    python examples/bert_fine_tuning.py [--pretrain-steps 150] [--finetune-steps 60] [--device cuda:0]
"""
import torch

from _common import backend_for, parser

from rustral_b200.core import ForwardCtx
from rustral_b200.nn import CrossEntropyLoss, LinearBuilder, TransformerEncoder, TransformerEncoderConfig
from rustral_b200.optim import Adam

PAD, CLS, MASK, FIRST = 0, 1, 2, 3
VOCAB, SEQ = 40, 16


def sequences(n, g):
    """Topic 0 prefers the lower half of the vocabulary, topic 1 the upper half; position 0 is <cls>."""
    topic = torch.randint(0, 2, (n,), generator=g)
    half = (VOCAB - FIRST) // 2
    own = torch.randint(0, half, (n, SEQ), generator=g) + FIRST + topic[:, None] * half
    other = torch.randint(FIRST, VOCAB, (n, SEQ), generator=g)
    ids = torch.where(torch.rand(n, SEQ, generator=g) < 0.85, own, other)
    ids[:, 0] = CLS
    return ids, topic


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--pretrain-steps", type=int, default=150)
    ap.add_argument("--finetune-steps", type=int, default=60)
    a = ap.parse_args(argv)
    backend = backend_for(a.device)
    dev = backend.device()
    cfg = TransformerEncoderConfig(d_model=48, num_heads=4, num_layers=2, ff_dim=96, dropout=0.0, max_seq_len=SEQ, vocab_size=VOCAB)
    enc = TransformerEncoder.new(backend, cfg, seed=a.seed)
    with torch.no_grad():
        enc.token_embedding.embed.tensor.mul_(10.0)
    mlm_head = LinearBuilder(cfg.d_model, VOCAB).with_bias().seed(a.seed + 1).build(backend)
    ce = CrossEntropyLoss()
    g = torch.Generator().manual_seed(a.seed)

    # ---- stage 1: masked-token prediction --------------------------------------------------------------------------
    opt = Adam(lr=3e-3)
    params = enc.parameters() + mlm_head.parameters()
    for step in range(a.pretrain_steps):
        ids, _ = sequences(64, g)
        mask = (torch.rand(ids.shape, generator=g) < 0.15) & (ids != CLS)
        mask[:, 1] |= ~mask.any(1)                                   # at least one masked position per row
        corrupted = torch.where(mask, torch.full_like(ids, MASK), ids).to(dev)
        for p in params:
            p.zero_grad()
        h = enc.forward(corrupted, ForwardCtx.train(backend))
        logits = mlm_head(h[mask.to(dev)].contiguous(), ForwardCtx.train(backend))
        loss = ce(logits.float(), ids.to(dev)[mask.to(dev)])
        loss.backward()
        opt.step(params)
        if step % 50 == 0 or step == a.pretrain_steps - 1:
            print(f"pre-train step {step}: masked-token loss {float(loss.detach()):.3f}")
    mlm_loss = float(loss.detach())

    # ---- stage 2: classification head on <cls>, encoder at a tenth of the head's learning rate -------------------
    clf = LinearBuilder(cfg.d_model, 2).with_bias().seed(a.seed + 2).scale(0.0).zero_bias().build(backend)   # starts undecided
    opt_head, opt_enc = Adam(lr=5e-3), Adam(lr=5e-4)
    test_ids, test_y = sequences(256, g)

    def accuracy():
        with torch.no_grad():
            ctx = ForwardCtx.inference()
            return float((clf(enc.cls_token(test_ids.to(dev), ctx).contiguous(), ctx).float().argmax(-1).cpu() == test_y).float().mean())
    before = accuracy()
    for step in range(a.finetune_steps):
        ids, y = sequences(32, g)
        for p in enc.parameters() + clf.parameters():
            p.zero_grad()
        ctx = ForwardCtx.train(backend)
        loss = ce(clf(enc.cls_token(ids.to(dev), ctx).contiguous(), ctx).float(), y.to(dev))
        loss.backward()
        opt_head.step(clf.parameters())
        opt_enc.step(enc.parameters())
    after = accuracy()
    print(f"fine-tuning: topic accuracy {before:.3f} -> {after:.3f}")
    return {"mlm_loss": mlm_loss, "accuracy_before": before, "accuracy_after": after}


if __name__ == "__main__":
    main()
