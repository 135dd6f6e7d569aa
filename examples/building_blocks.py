"""A tour of the layer library: every block is constructed from the backend, run once, and its output shape and
parameter count printed; then blocks are composed into a small pre-norm transformer by hand
(crates/nn/examples/building_blocks.rs, transformer_composition.rs).

    python examples/building_blocks.py [--device cuda:0]
"""
import torch

from _common import backend_for, parser

from rustral_b200.core import ForwardCtx
from rustral_b200.nn import (BatchNorm, Conv2d, Conv2dConfig, Dropout, DropoutConfig, Embedding, ExpertLayer, GruCell, LayerNorm,
                             LinearBuilder, LstmCell, MoEConfig, MultiHeadAttention, PositionalEncoding, RMSNorm, Sequential,
                             SwiGLUFeedForward, TransformerEncoderBlock, causal_mask)


def main(argv=None):
    a = parser(__doc__).parse_args(argv)
    backend = backend_for(a.device)
    dev, dt = backend.device(), backend.dtype
    ctx = ForwardCtx.inference()
    g = torch.Generator().manual_seed(a.seed)
    rows = []

    def show(name, module, out):
        n = module.num_parameters() if hasattr(module, "num_parameters") else 0
        shape = tuple(out.shape) if hasattr(out, "shape") else out
        rows.append((name, shape, n))
        print(f"{name:<28} -> {str(shape):<18} {n:>7} parameters")

    x = torch.randn(4, 10, 32, generator=g).to(dev, dt)                       # [batch, sequence, features]
    lin = LinearBuilder(32, 64).with_bias().seed(1).build(backend)
    show("Linear 32->64", lin, lin(x, ctx))
    fused = LinearBuilder(32, 64).with_bias().seed(2).activation("gelu").build(backend)
    show("Linear + GELU (one kernel)", fused, fused(x, ctx))
    emb = Embedding.new(backend, 100, 32)
    ids = torch.randint(0, 100, (4, 10), generator=g).to(dev)
    show("Embedding 100x32", emb, emb(ids, ctx))
    pe = PositionalEncoding(32, 64, dev, dt)
    show("PositionalEncoding", pe, pe(x, ctx))
    show("LayerNorm", LayerNorm.new(backend, 32), LayerNorm.new(backend, 32)(x, ctx))
    rms = RMSNorm.new(backend, 32)
    show("RMSNorm", rms, rms(x, ctx))
    bn = BatchNorm.new(backend, 32)
    show("BatchNorm (inference)", bn, bn(x[:, 0].contiguous(), ctx))
    drop = Dropout(DropoutConfig(0.5))
    kept = float((drop(torch.ones(64, 64, device=dev, dtype=dt), ForwardCtx.train(backend, seed=3)) != 0).float().mean())
    show(f"Dropout 0.5 (kept {kept:.2f})", drop, (64, 64))
    mha = MultiHeadAttention.new(backend, 32, 4)
    show("MultiHeadAttention 4 heads", mha, mha(x, ctx))
    show("  .. with a causal mask", mha, mha.forward(x, ctx, causal_mask(backend, 10)))
    ffn = SwiGLUFeedForward.new(backend, 32, 96)
    show("SwiGLU feed-forward", ffn, ffn(x, ctx))
    block = TransformerEncoderBlock.new(backend, 32, 4, 64)
    show("TransformerEncoderBlock", block, block(x, ctx))
    moe = ExpertLayer.new(backend, MoEConfig(32, 4, 64, 2))
    show("MoE 4 experts top-2", moe, moe(x, ctx).output)
    conv = Conv2d.new(backend, Conv2dConfig(8, 3, 3, in_channels=3))
    show("Conv2d 3->8, 3x3", conv, conv(torch.randn(2, 3, 12, 12, generator=g).to(dev, dt), ctx))
    lstm = LstmCell.new(backend, 32, 48)
    seq = x.transpose(0, 1).contiguous()                                       # recurrent cells take [time, batch, features]
    show("LSTM over 10 steps", lstm, lstm.forward_sequence(seq, ctx)[0])
    gru = GruCell.new(backend, 32, 48)
    show("GRU over 10 steps", gru, gru.forward_sequence(seq, ctx)[0])

    # composition: embedding + positions -> two encoder blocks -> norm -> classifier over the mean token
    body = Sequential(TransformerEncoderBlock.new(backend, 32, 4, 64, seed=10), TransformerEncoderBlock.new(backend, 32, 4, 64, seed=20),
                      LayerNorm.new(backend, 32))
    head = LinearBuilder(32, 5).with_bias().seed(30).build(backend)
    h = body(pe(emb(ids, ctx), ctx), ctx)
    logits = head(h.mean(1).contiguous(), ctx)
    total = emb.num_parameters() + body.num_parameters() + head.num_parameters()
    print(f"composed classifier: ids {tuple(ids.shape)} -> logits {tuple(logits.shape)}, {total} parameters, "
          f"first names {[n for n, _ in body.named_parameters()][:3]}")
    return {"rows": rows, "logits_shape": tuple(logits.shape), "total": total}


if __name__ == "__main__":
    main()
