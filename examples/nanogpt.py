"""A character-level GPT: decoder-only transformer trained on an embedded text and sampled with the cached serving path
off (full re-forward), then the same weights saved and re-loaded (crates/candle-backend/examples/nanogpt.rs,
crates/nn/examples/gpt_training.rs, transformer_gpt_decoder.rs).  `examples/pretrain_lm.py` is the full-size counterpart
on the fused engine.

    python examples/nanogpt.py [--steps 200] [--d-model 64] [--layers 2] [--device cuda:0]
"""
import math

import torch

from _common import backend_for, parser
from _synthetic import TEXT

from rustral_b200.core import ForwardCtx
from rustral_b200.nn import CrossEntropyLoss, TransformerDecoder, TransformerDecoderConfig
from rustral_b200.optim import AdamW, WarmupCosine
from rustral_b200.runtime.model_io import load_model, save_model


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--block", type=int, default=32)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--d-model", type=int, default=64)
    ap.add_argument("--layers", type=int, default=2)
    a = ap.parse_args(argv)
    backend = backend_for(a.device)
    dev = backend.device()
    chars = sorted(set(TEXT))
    stoi = {c: i for i, c in enumerate(chars)}
    data = torch.tensor([stoi[c] for c in TEXT], device=dev)
    cfg = TransformerDecoderConfig(d_model=a.d_model, num_heads=4, num_layers=a.layers, ff_dim=4 * a.d_model, dropout=0.0,
                                   max_seq_len=a.block + 64, vocab_size=len(chars))
    model = TransformerDecoder.new(backend, cfg, seed=a.seed)
    with torch.no_grad():
        model.token_embedding.embed.tensor.mul_(10.0)          # N(0, 0.02) would be drowned by the unit-size positions
    opt = AdamW(lr=3e-3, weight_decay=0.01, max_grad_norm=1.0)
    sched = WarmupCosine(3e-3, 3e-4, 10, a.steps).attach(opt)
    ce = CrossEntropyLoss()
    g = torch.Generator().manual_seed(a.seed)
    first = last = None
    for step in range(a.steps):
        starts = torch.randint(0, len(data) - a.block - 1, (a.batch,), generator=g).tolist()
        x = torch.stack([data[s:s + a.block] for s in starts])
        y = torch.stack([data[s + 1:s + a.block + 1] for s in starts])
        model.zero_grad()
        loss = ce(model.forward(x, ForwardCtx.train(backend)).reshape(-1, len(chars)).float(), y.reshape(-1))
        loss.backward()
        opt.step(model.parameters())
        sched.step()
        last = float(loss.detach())
        first = last if first is None else first
        if step % 50 == 0 or step == a.steps - 1:
            print(f"step {step}: loss {last:.3f}  (uniform {math.log(len(chars)):.3f})  lr {opt.lr:.2e}")
    ctx = ForwardCtx.inference()
    ids = [stoi[c] for c in "the "]
    with torch.no_grad():
        for _ in range(60):
            ids.append(model.generate_token(torch.tensor(ids[-a.block:], device=dev), ctx))
    text = "".join(chars[i] for i in ids)
    print("greedy continuation:", text)
    blob = save_model(model)
    twin = TransformerDecoder.new(backend, cfg, seed=a.seed + 1)
    load_model(twin, blob)
    probe = torch.tensor([ids[:16]], device=dev)
    with torch.no_grad():
        same = torch.equal(model.forward(probe, ctx), twin.forward(probe, ctx))
    print(f"saved {len(blob)} bytes; re-loaded copy gives identical logits: {same}")
    return {"loss_first": first, "loss_last": last, "text": text, "roundtrip": same}


if __name__ == "__main__":
    main()
