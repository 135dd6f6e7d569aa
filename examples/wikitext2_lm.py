"""WikiText-2 word-level language model trained through the tape trainer (crates/runtime/examples/wikitext2_lm.rs).

Model: token embedding + positions -> N causal pre-norm transformer layers -> final norm -> vocabulary logits.
Every window of `block_size` tokens is trained on ALL of its next-token targets in one batched forward (the reference
predicts one token per window from the last position); dev perplexity is exp(mean next-token loss in nats) over the
validation windows.  Writes `manifest.json` and `vocab.txt` to `--out-dir`.

    python examples/wikitext2_lm.py --quick --block-size 16 --d-model 32 --num-heads 2 --ffn-dim 64 --num-layers 1
    RUSTRAL_DATASET_OFFLINE=1 python examples/wikitext2_lm.py   # wiki.{train,valid,test}.tokens (or {train,valid,
                                                                # test}.txt) under $RUSTRAL_CACHE_DIR/datasets/wikitext-2/
"""
import argparse
import math
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rustral_b200 import ops                                                                  # noqa: E402
from rustral_b200.bench.manifest import validate_manifest, write_manifest                    # noqa: E402
from rustral_b200.core import CpuBackend, ForwardCtx                                          # noqa: E402
from rustral_b200.core.module import Module, Trainable                                        # noqa: E402
from rustral_b200.data.corpora import load_wikitext2                                          # noqa: E402
from rustral_b200.data.fetch import fnv1a64                                                   # noqa: E402
from rustral_b200.data.tokenizer import WordLevelConfig, WordLevelTokenizer                   # noqa: E402
from rustral_b200.nn.transformer import TransformerDecoder, TransformerDecoderConfig          # noqa: E402
from rustral_b200.optim import Adam                                                           # noqa: E402
from rustral_b200.runtime.tape_trainer import SupervisedTapeModel, Trainer                    # noqa: E402

MAX_VOCAB = 16384
DEFAULT_SEED = 0xC0FFEE


class WordLM(Module, Trainable, SupervisedTapeModel):
    def __init__(self, backend, vocab_size, block_size, d_model, num_heads, ffn_dim, num_layers, seed):
        cfg = TransformerDecoderConfig(d_model, num_heads, num_layers, ffn_dim, dropout=0.0, max_seq_len=block_size,
                                       vocab_size=vocab_size)
        self.decoder = TransformerDecoder.new(backend, cfg, seed=seed % (1 << 31))
        self._device, self._vocab = backend.device(), vocab_size

    def forward(self, ids, ctx):
        """Logits flattened to [B * S, vocab] so the loss is one cross entropy over every position."""
        logits = self.decoder.forward(torch.as_tensor(ids, dtype=torch.int64, device=self._device), ctx)
        return logits.reshape(-1, self._vocab)

    def forward_tape(self, x, tape, ctx):
        return tape.apply("word_lm", lambda: self.forward(x, ctx))

    def loss_tape(self, logits, y, tape, ctx):
        return tape.cross_entropy_loss(logits, y.reshape(-1))

    def collate(self, xs):
        return torch.tensor(xs, dtype=torch.int64, device=self._device)

    def collate_targets(self, ys):
        return torch.tensor(ys, dtype=torch.int64, device=self._device)


def windows(ids, block):
    """Non-overlapping (inputs, next-token targets) windows."""
    return [(ids[i:i + block], ids[i + 1:i + block + 1]) for i in range(0, len(ids) - block - 1, block)]


def evaluate(model, data, batch):
    ctx = ForwardCtx.inference()
    total, n = 0.0, 0
    with torch.no_grad():
        for i in range(0, len(data), batch):
            chunk = data[i:i + batch]
            logits = model.forward(model.collate([x for x, _ in chunk]), ctx)
            y = model.collate_targets([y for _, y in chunk]).reshape(-1)
            total += float(ops.cross_entropy(logits, y)) * y.numel()
            n += y.numel()
    return total / max(1, n)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--paper", action="store_true", help="block 64, d_model 128, FFN 256, 5 epochs, 500k training tokens")
    ap.add_argument("--overfit-tiny", action="store_true", help="train and evaluate on the first 8 windows")
    ap.add_argument("--seed", type=int, default=DEFAULT_SEED)
    ap.add_argument("--block-size", type=int)
    ap.add_argument("--d-model", type=int)
    ap.add_argument("--num-heads", type=int, default=4)
    ap.add_argument("--ffn-dim", type=int)
    ap.add_argument("--num-layers", type=int, default=2)
    ap.add_argument("--epochs", type=int)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--lr", type=float)
    ap.add_argument("--train-tokens", type=int, help="cap on the training tokens used (0 = all)")
    ap.add_argument("--train-windows", type=int, default=0, help="cap on the training windows (0 = all)")
    ap.add_argument("--eval-windows", type=int, default=0, help="cap on the validation windows (0 = all)")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--out-dir", default="out/wikitext2")
    a = ap.parse_args(argv)
    quick = a.quick and not a.paper
    block = a.block_size or (64 if a.paper else 32)
    d_model = a.d_model or (128 if a.paper else 64)
    ffn_dim = a.ffn_dim or (256 if a.paper else 128)
    epochs = a.epochs or (5 if a.paper else 60 if a.overfit_tiny else 1)
    lr = a.lr or (3e-3 if a.overfit_tiny else 1e-3 if a.paper else 5e-4)
    cap = a.train_tokens if a.train_tokens is not None else (4000 if quick else 500000 if a.paper else 50000)
    if d_model % a.num_heads:
        raise SystemExit(f"--d-model ({d_model}) must be divisible by --num-heads ({a.num_heads})")
    os.makedirs(a.out_dir, exist_ok=True)

    train_text, valid_text = load_wikitext2("train"), load_wikitext2("valid")
    digest = fnv1a64((train_text + "\n" + valid_text).encode("utf-8"))
    tok = WordLevelTokenizer.fit_from_iter([train_text], WordLevelConfig(lowercase=True, max_vocab=MAX_VOCAB))
    tok.save_vocab(os.path.join(a.out_dir, "vocab.txt"))
    train_ids = tok.encode(train_text)
    if cap:
        train_ids = train_ids[:cap]
    train = windows(train_ids, block)
    valid = windows(tok.encode(valid_text)[:cap or None], block)
    n_train_all, n_valid_all = len(train), len(valid)
    if a.train_windows:
        train = train[:a.train_windows]
    if a.overfit_tiny:
        train = train[:8]
        valid = train
    if a.eval_windows:
        valid = valid[:a.eval_windows]
    if not train or not valid:
        raise SystemExit(f"corpus too small for block size {block}: {len(train_ids)} training tokens")

    if a.device == "cpu":
        backend = CpuBackend()
    else:
        from rustral_b200.core import B200Backend
        backend = B200Backend(a.device)
    model = WordLM(backend, len(tok.vocab), block, d_model, a.num_heads, ffn_dim, a.num_layers, a.seed)
    total_params = model.num_parameters()
    print(f"wikitext2: tokens={len(train_ids)} windows={len(train)} valid_windows={len(valid)} vocab={len(tok.vocab)} "
          f"params={total_params} epochs={epochs} lr={lr}")
    t0 = time.perf_counter()
    report = Trainer.regression(Adam(lr=lr)).epochs(epochs).batch_size(a.batch).shuffle(True).seed(a.seed % (1 << 31)) \
        .fit(backend, model, train)
    elapsed = time.perf_counter() - t0
    for e in report.epochs[-5:]:
        print(f"epoch {e.epoch}: loss={e.mean_loss:.4f} ({e.elapsed:.2f}s)")
    val_loss = evaluate(model, valid, a.batch)
    val_ppl = math.exp(min(val_loss, 50.0))
    print(f"dev: loss={val_loss:.4f} nats, perplexity={val_ppl:.2f}; {report.throughput.examples_per_sec:.1f} windows/s")
    doc = write_manifest(os.path.join(a.out_dir, "manifest.json"), "wikitext2_word_lm", {
        "model_type": "transformer_lm", "seed": a.seed, "block_size": block, "d_model": d_model, "num_heads": a.num_heads,
        "ffn_dim": ffn_dim, "num_layers": a.num_layers, "total_params": total_params, "max_vocab": MAX_VOCAB,
        "vocab_size": len(tok.vocab), "epochs": epochs, "batch_size": a.batch, "learning_rate": lr,
        "train_tokens_used": len(train_ids), "train_windows": n_train_all, "train_windows_used": len(train),
        "valid_windows": n_valid_all, "eval_windows_used": len(valid), "dataset_hash_fnv1a": f"{digest:016x}",
        "dev_loss_nats": val_loss, "dev_perplexity": val_ppl, "windows_per_sec": report.throughput.examples_per_sec,
        "tokens_per_sec": report.throughput.examples_per_sec * block, "train_elapsed_sec": elapsed,
        "dataset": "WikiText-2 raw v1", "tokenizer": "WordLevelTokenizer (whitespace, lowercased)",
        "device": str(backend.device()), "quick_mode": quick, "paper_mode": a.paper, "overfit_tiny": a.overfit_tiny,
        "lr_schedule_note": "constant"},
        {"epoch_losses": [e.mean_loss for e in report.epochs], "targets_per_window": block,
         "uniform_perplexity": float(len(tok.vocab))})
    problems = validate_manifest(doc)
    if problems:
        raise SystemExit("\n".join(problems))
    print(f"wrote {os.path.join(a.out_dir, 'manifest.json')}")
    return doc


if __name__ == "__main__":
    main()
