"""SST-2 sentiment classifier trained through the tape trainer (crates/runtime/examples/sst2_classifier.rs).

Model: token embedding + sinusoidal positions -> N pre-norm transformer encoder layers -> masked mean pool over the
non-padding positions -> Linear(d_model, 2).  Word-level tokenizer (whitespace, lower-cased, at most 8192 entries)
fitted on the training split.  Writes `manifest.json` (hyper-parameters, dataset hash and sizes, dev loss / accuracy,
throughput, label / confusion diagnostics) and `vocab.txt` to `--out-dir`.

    python examples/sst2_classifier.py                      # 3 epochs on the full training set
    python examples/sst2_classifier.py --quick              # 256 examples, 1 epoch: seconds
    RUSTRAL_DATASET_OFFLINE=1 python examples/sst2_classifier.py    # train.jsonl / dev.jsonl (or .tsv) pre-staged
                                                                    # under $RUSTRAL_CACHE_DIR/datasets/sst2/
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rustral_b200.bench.manifest import validate_manifest, write_manifest                    # noqa: E402
from rustral_b200.core import CpuBackend, ForwardCtx                                          # noqa: E402
from rustral_b200.core.module import Module, Trainable                                        # noqa: E402
from rustral_b200.data.corpora import load_sst2                                               # noqa: E402
from rustral_b200.data.fetch import fnv1a64                                                   # noqa: E402
from rustral_b200.data.tokenizer import WordLevelConfig, WordLevelTokenizer                   # noqa: E402
from rustral_b200.nn.linear import LinearBuilder                                              # noqa: E402
from rustral_b200.nn.transformer import TransformerEncoder, TransformerEncoderConfig          # noqa: E402
from rustral_b200.optim import Adam, Sgd                                                      # noqa: E402
from rustral_b200.runtime.tape_trainer import SupervisedTapeModel, Trainer                    # noqa: E402

MAX_VOCAB = 8192
DEFAULT_SEED = 0xC0FFEE


class Sst2Model(Module, Trainable, SupervisedTapeModel):
    def __init__(self, backend, vocab_size, seq_len, d_model, num_heads, ffn_dim, num_layers, pad_id, seed):
        cfg = TransformerEncoderConfig(d_model, num_heads, num_layers, ffn_dim, dropout=0.0, max_seq_len=seq_len,
                                       vocab_size=vocab_size)
        self.encoder = TransformerEncoder.new(backend, cfg, seed=seed % (1 << 31))
        self.head = LinearBuilder(d_model, 2).with_bias().seed(seed % (1 << 31) + 1).scale(0.02).zero_bias().build(backend)
        self._pad_id, self._seq_len, self._device = pad_id, seq_len, backend.device()

    def forward(self, ids, ctx):
        ids = torch.as_tensor(ids, dtype=torch.int64, device=self._device)
        keep = (ids != self._pad_id).to(torch.float32)
        h = self.encoder.forward(ids, ctx)                                     # [B, S, d]
        w = (keep / keep.sum(-1, keepdim=True).clamp_min(1.0)).to(h.dtype)     # masked mean over real tokens
        pooled = torch.bmm(w.unsqueeze(1), h).squeeze(1)
        return self.head(pooled.contiguous(), ctx)

    def forward_tape(self, x, tape, ctx):
        return tape.apply("sst2_encoder_classifier", lambda: self.forward(x, ctx))

    def collate(self, xs):
        return torch.tensor(xs, dtype=torch.int64, device=self._device)

    def collate_targets(self, ys):
        return torch.tensor(ys, dtype=torch.int64, device=self._device)


def encode(tok, text, seq_len):
    ids = tok.encode(text)[:seq_len]
    return ids + [tok.vocab.pad_id] * (seq_len - len(ids))


def evaluate(model, data, batch):
    """Mean loss, accuracy and the diagnostics block of the manifest over `data` = [(ids, label)]."""
    ctx = ForwardCtx.inference()
    loss_sum, conf, hist = 0.0, [[0, 0], [0, 0]], [0] * 10
    with torch.no_grad():
        for i in range(0, len(data), batch):
            chunk = data[i:i + batch]
            logits = model.forward(model.collate([x for x, _ in chunk]), ctx).float()
            y = model.collate_targets([y for _, y in chunk])
            logp = torch.log_softmax(logits, -1)
            loss_sum += float(-logp.gather(1, y[:, None]).sum())
            pred = logits.argmax(-1)
            for t, p, pp in zip(y.tolist(), pred.tolist(), logp[:, 1].exp().tolist()):
                conf[t][p] += 1
                hist[min(9, int(pp * 10))] += 1
    n = max(1, len(data))
    return {"loss": loss_sum / n, "accuracy": (conf[0][0] + conf[1][1]) / n, "confusion": conf, "hist": hist}


def parity_one_step(model, rows, lr, a, seq_len, d_model, ffn_dim):
    """Runs one training step on `rows` and writes everything an outside implementation needs to repeat it: the batch,
    the hyper-parameters, every parameter before the step, the logits, the loss, every gradient and every parameter
    after one Adam step (`python -m rustral_b200.bench.sst2_parity <dump>` repeats it in plain PyTorch and compares;
    the reference's counterpart is scripts/eval/sst2_parity_one_step.py)."""
    from rustral_b200.nn.loss import CrossEntropyLoss
    ctx = ForwardCtx.train()
    ids = model.collate([x for x, _ in rows])
    labels = model.collate_targets([y for _, y in rows])
    named = list(model.named_parameters())
    before = {n: p.tensor.detach().float().cpu().reshape(-1).tolist() for n, p in named}
    shapes = {n: list(p.tensor.shape) for n, p in named}
    model.zero_grad()
    logits = model.forward(ids, ctx)
    loss = CrossEntropyLoss()(logits.float(), labels)
    loss.backward()
    grads = {n: (p.tensor.grad.detach().float().cpu().reshape(-1).tolist() if p.tensor.grad is not None else None) for n, p in named}
    Adam(lr=lr).step([p for _, p in named])
    after = {n: p.tensor.detach().float().cpu().reshape(-1).tolist() for n, p in named}
    path = a.parity_dump or os.path.join(a.out_dir, "parity.json")
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "w") as f:
        json.dump({"task": "sst2_parity_one_step", "ids": ids.cpu().tolist(), "labels": labels.cpu().tolist(),
                   "config": {"seq_len": seq_len, "d_model": d_model, "num_heads": a.num_heads, "ffn_dim": ffn_dim,
                              "num_layers": a.num_layers, "pad_id": model._pad_id, "lr": lr, "layer_norm_eps": 1e-5,
                              "adam": {"beta1": 0.9, "beta2": 0.999, "eps": 1e-8}, "gelu": "tanh"},
                   "shapes": shapes, "params_before": before, "logits": logits.detach().float().cpu().reshape(-1).tolist(),
                   "loss": float(loss), "grads": grads, "params_after": after}, f)
    print(f"parity: batch={len(rows)} loss={float(loss):.6f}; wrote {path}")
    return path


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--paper", action="store_true", help="seq 64, d_model 128, FFN 256, 10 epochs")
    ap.add_argument("--overfit-32", action="store_true", help="train and evaluate on the first 32 examples")
    ap.add_argument("--sgd", action="store_true")
    ap.add_argument("--seed", type=int, default=DEFAULT_SEED)
    ap.add_argument("--num-layers", type=int, default=2)
    ap.add_argument("--epochs", type=int)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--lr", type=float)
    ap.add_argument("--seq-len", type=int)
    ap.add_argument("--d-model", type=int)
    ap.add_argument("--num-heads", type=int, default=4)
    ap.add_argument("--ffn-dim", type=int)
    ap.add_argument("--vocab", help="reuse a vocab.txt instead of fitting one")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--out-dir", default="out/sst2")
    ap.add_argument("--parity-one-step", action="store_true",
                    help="one forward / backward / Adam step on the first --parity-batch examples, dumped for an independent check")
    ap.add_argument("--parity-batch", type=int, default=8)
    ap.add_argument("--parity-dump", default=None, help="where the one-step record goes (default <out-dir>/parity.json)")
    a = ap.parse_args(argv)
    quick = a.quick and not a.paper
    epochs = a.epochs or (1 if quick else 10 if a.paper else 40 if a.overfit_32 else 3)
    lr = a.lr or (1e-3 if a.paper else 3e-3 if a.overfit_32 else 5e-4)
    seq_len = a.seq_len or (64 if a.paper else 32)
    d_model = a.d_model or (128 if a.paper else 64)
    ffn_dim = a.ffn_dim or (256 if a.paper else 128)
    if d_model % a.num_heads:
        raise SystemExit(f"--d-model ({d_model}) must be divisible by --num-heads ({a.num_heads})")
    os.makedirs(a.out_dir, exist_ok=True)

    train, dev = load_sst2("train"), load_sst2("dev")
    if quick:
        train, dev = train[:256], dev[:256]
    if a.overfit_32:
        train = train[:32]
        dev = train
    digest = fnv1a64("\n".join(f"{e.label}\t{e.text}" for e in train + dev).encode("utf-8"))
    tok = (WordLevelTokenizer.from_vocab_file(a.vocab) if a.vocab else
           WordLevelTokenizer.fit_from_iter((e.text for e in train), WordLevelConfig(lowercase=True, max_vocab=MAX_VOCAB)))
    tok.save_vocab(os.path.join(a.out_dir, "vocab.txt"))
    tr = [(encode(tok, e.text, seq_len), e.label) for e in train]
    dv = [(encode(tok, e.text, seq_len), e.label) for e in dev]

    if a.device == "cpu":
        backend = CpuBackend()
    else:
        from rustral_b200.core import B200Backend
        backend = B200Backend(a.device)
    model = Sst2Model(backend, len(tok.vocab), seq_len, d_model, a.num_heads, ffn_dim, a.num_layers, tok.vocab.pad_id, a.seed)
    total_params = model.num_parameters()
    print(f"sst2: train={len(tr)} dev={len(dv)} vocab={len(tok.vocab)} params={total_params} epochs={epochs} lr={lr} "
          f"offline={os.environ.get('RUSTRAL_DATASET_OFFLINE') == '1'}")
    if a.parity_one_step:
        return parity_one_step(model, tr[:a.parity_batch], lr, a, seq_len, d_model, ffn_dim)
    opt = Sgd(lr=lr) if a.sgd else Adam(lr=lr)
    t0 = time.perf_counter()
    report = Trainer.classification(opt).epochs(epochs).batch_size(a.batch).shuffle(True).seed(a.seed % (1 << 31)) \
        .fit(backend, model, tr)
    elapsed = time.perf_counter() - t0
    for e in report.epochs:
        print(f"epoch {e.epoch}: loss={e.mean_loss:.4f} acc={e.accuracy:.3f} ({e.elapsed:.2f}s)")
    ev = evaluate(model, dv, a.batch)
    print(f"dev: loss={ev['loss']:.4f} acc={ev['accuracy']:.3f}; {report.throughput.examples_per_sec:.1f} samples/s")

    def counts(rows):
        c = [0, 0]
        for _, y in rows:
            c[y] += 1
        return c
    l2 = {}
    for name, p in model.named_parameters():
        key = name.split(".")[0] if not name.startswith("encoder.layers") else ".".join(name.split(".")[:3])
        l2[key] = l2.get(key, 0.0) + float(p.tensor.detach().float().pow(2).sum())
    diagnostics = {"train_label_counts": counts(tr), "dev_label_counts": counts(dv), "dev_confusion_matrix": ev["confusion"],
                   "dev_predicted_counts": [ev["confusion"][0][0] + ev["confusion"][1][0], ev["confusion"][0][1] + ev["confusion"][1][1]],
                   "dev_positive_prob_hist": ev["hist"], "epoch_losses": [e.mean_loss for e in report.epochs],
                   "param_l2_by_prefix": {k: v ** 0.5 for k, v in l2.items()}}
    doc = write_manifest(os.path.join(a.out_dir, "manifest.json"), "sst2_classifier", {
        "model_type": "transformer_encoder", "seed": a.seed, "seq_len": seq_len, "d_model": d_model,
        "num_heads": a.num_heads, "ffn_dim": ffn_dim, "num_layers": a.num_layers, "total_params": total_params,
        "max_vocab": MAX_VOCAB, "vocab_size": len(tok.vocab), "epochs": epochs, "batch_size": a.batch,
        "learning_rate": lr, "optimizer": "sgd" if a.sgd else "adam", "train_examples": len(tr), "dev_examples": len(dv),
        "dataset_hash_fnv1a": f"{digest:016x}", "dev_loss": ev["loss"], "dev_accuracy": ev["accuracy"],
        "samples_per_sec": report.throughput.examples_per_sec, "train_elapsed_sec": elapsed,
        "dataset": "SST-2 (binary, HuggingFace SetFit/sst2 mirror)",
        "tokenizer": "WordLevelTokenizer (whitespace, lowercased)", "device": str(backend.device()),
        "quick_mode": quick, "paper_mode": a.paper, "overfit_32": a.overfit_32, "lr_schedule_note": "constant"}, diagnostics)
    problems = validate_manifest(doc)
    if problems:
        raise SystemExit("\n".join(problems))
    print(f"wrote {os.path.join(a.out_dir, 'manifest.json')}")
    return doc


if __name__ == "__main__":
    main()
