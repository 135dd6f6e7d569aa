"""Character-level next-character LM: the whole training spine in one command, no downloads
(crates/runtime/examples/emnlp_char_lm.rs).

An in-file public-domain text excerpt -> character vocabulary -> deterministic train / validation split of
(8 previous characters -> next character) samples -> Embedding(vocab, 16) + Linear(8 * 16, vocab) trained with
`TapeTrainer.fit_classification` (Adam, 12 epochs) -> validation loss / accuracy -> strict save / load round trip
with logit equality -> greedy generation from a fixed prompt.

    python examples/emnlp_char_lm.py
    python examples/emnlp_char_lm.py --determinism-check      # three runs from one seed must agree bit for bit;
                                                              # writes emnlp_determinism_report.json to --out-dir
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rustral_b200.core import CpuBackend, ForwardCtx                           # noqa: E402
from rustral_b200.core.module import Module, Trainable                         # noqa: E402
from rustral_b200.nn.embedding import Embedding                                # noqa: E402
from rustral_b200.nn.linear import LinearBuilder                               # noqa: E402
from rustral_b200.optim import Adam                                            # noqa: E402
from rustral_b200.runtime.model_io import load_model, save_model               # noqa: E402
from rustral_b200.runtime.tape_trainer import SupervisedTapeModel, TapeTrainer, TapeTrainerConfig   # noqa: E402

CORPUS = (
    "To be, or not to be, that is the question:\n"
    "Whether 'tis nobler in the mind to suffer\n"
    "The slings and arrows of outrageous fortune,\n"
    "Or to take arms against a sea of troubles\n"
    "And by opposing end them. To die, to sleep,\n"
    "No more; and by a sleep to say we end\n"
    "The heart-ache and the thousand natural shocks\n"
    "That flesh is heir to: 'tis a consummation\n"
    "Devoutly to be wish'd. To die, to sleep;\n"
    "To sleep, perchance to dream. Ay, there's the rub,\n"
    "For in that sleep of death what dreams may come,\n"
    "When we have shuffled off this mortal coil,\n"
    "Must give us pause.\n")
BLOCK_SIZE, EMBED_DIM, EPOCHS, BATCH_SIZE, LEARNING_RATE = 8, 16, 12, 16, 5e-3
VAL_FRACTION, GENERATE_LEN, PROMPT = 0.15, 80, "To be"


class CharVocab:
    def __init__(self, text: str):
        self.chars = sorted(set(text))
        self.index = {c: i for i, c in enumerate(self.chars)}

    def __len__(self):
        return len(self.chars)

    def encode(self, c: str) -> int:
        return self.index.get(c, 0)

    def decode(self, i: int) -> str:
        return self.chars[i] if 0 <= i < len(self.chars) else "?"


def build_samples(ids, block):
    return [(ids[i:i + block], ids[i + block]) for i in range(len(ids) - block)]


class CharLM(Module, Trainable, SupervisedTapeModel):
    def __init__(self, backend, vocab: int, seed: int):
        self.embed = Embedding.new(backend, vocab, EMBED_DIM, seed)
        self.head = LinearBuilder(BLOCK_SIZE * EMBED_DIM, vocab).with_bias().seed(seed + 1).scale(0.1).zero_bias().build(backend)
        self._device = backend.device()

    def forward(self, ids, ctx):
        ids = torch.as_tensor(ids, dtype=torch.int64, device=self._device).reshape(-1, BLOCK_SIZE)
        e = self.embed(ids.reshape(-1), ctx).reshape(ids.shape[0], BLOCK_SIZE * EMBED_DIM)
        return self.head(e.contiguous(), ctx)

    def forward_tape(self, x, tape, ctx):
        return tape.apply("char_lm", lambda: self.forward(x, ctx))

    def collate(self, xs):
        return torch.tensor(xs, dtype=torch.int64, device=self._device)

    def collate_targets(self, ys):
        return torch.tensor(ys, dtype=torch.int64, device=self._device)

    def logits(self, ids):
        with torch.no_grad():
            return self.forward([list(ids)], ForwardCtx.inference())[0].float().cpu()


def generate_greedy(model, vocab, prompt: str, n: int) -> str:
    ids = [vocab.encode(c) for c in prompt]
    out = prompt
    for _ in range(n):
        window = ([0] * BLOCK_SIZE + ids)[-BLOCK_SIZE:]
        nxt = int(model.logits(window).argmax())
        ids.append(nxt)
        out += vocab.decode(nxt)
    return out


def validate(model, data):
    if not data:
        return float("nan"), float("nan")
    with torch.no_grad():
        logits = model.forward([x for x, _ in data], ForwardCtx.inference()).float().cpu()
    y = torch.tensor([t for _, t in data])
    loss = float(torch.nn.functional.cross_entropy(logits, y))
    return loss, float((logits.argmax(-1) == y).float().mean())


def train_once(seed: int, log: bool, device: str = "cpu") -> dict:
    if device == "cpu":
        backend = CpuBackend()
    else:
        from rustral_b200.core import B200Backend
        backend = B200Backend(device)
    vocab = CharVocab(CORPUS)
    samples = build_samples([vocab.encode(c) for c in CORPUS], BLOCK_SIZE)
    n_val = max(1, int(len(samples) * VAL_FRACTION))
    val_idx = set(range(0, len(samples), max(1, len(samples) // n_val)))       # every k-th sample: deterministic, spread out
    train = [s for i, s in enumerate(samples) if i not in val_idx]
    val = [s for i, s in enumerate(samples) if i in val_idx]
    model = CharLM(backend, len(vocab), seed)
    trainer = TapeTrainer(TapeTrainerConfig(epochs=EPOCHS, lr=LEARNING_RATE, batch_size=BATCH_SIZE, shuffle=True, seed=seed),
                          Adam(lr=LEARNING_RATE), backend)
    t0 = time.perf_counter()
    report = trainer.fit_classification(model, train)
    elapsed = time.perf_counter() - t0
    if log:
        for e in report.epochs:
            print(f"epoch {e.epoch:2d}: loss={e.mean_loss:.4f} acc={e.accuracy:.3f}")
    val_loss, val_acc = validate(model, val)
    blob = save_model(model)
    clone = CharLM(backend, len(vocab), seed + 999)
    load_model(clone, blob)
    probe = [vocab.encode(c) for c in "question"][:BLOCK_SIZE]
    roundtrip_ok = bool(torch.equal(model.logits(probe), clone.logits(probe)))
    text = generate_greedy(clone, vocab, PROMPT, GENERATE_LEN)
    return {"seed": seed, "vocab_size": len(vocab), "train_samples": len(train), "val_samples": len(val),
            "total_params": model.num_parameters(), "epoch_losses": [e.mean_loss for e in report.epochs],
            "train_accuracy": report.accuracy, "val_loss": val_loss, "val_accuracy": val_acc,
            "roundtrip_ok": roundtrip_ok, "generated": text, "checkpoint_bytes": len(blob),
            "samples_per_sec": report.throughput.examples_per_sec, "train_elapsed_sec": elapsed}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--determinism-check", action="store_true")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--out-dir", default=".")
    a = ap.parse_args(argv)
    if not a.determinism_check:
        r = train_once(a.seed, True, a.device)
        print(f"val: loss={r['val_loss']:.4f} acc={r['val_accuracy']:.3f}; save/load logits equal: {r['roundtrip_ok']}")
        print("generated:", json.dumps(r["generated"]))
        if not r["roundtrip_ok"]:
            raise SystemExit("checkpoint round trip changed the logits")
        return r
    keys = ("epoch_losses", "val_loss", "val_accuracy", "generated")
    runs = [train_once(a.seed, False, a.device) for _ in range(3)]
    all_equal = all(all(r[k] == runs[0][k] for k in keys) for r in runs[1:])
    report = {"seed": a.seed, "runs": [{k: r[k] for k in keys} for r in runs], "all_equal": all_equal, "device": a.device}
    os.makedirs(a.out_dir, exist_ok=True)
    path = os.path.join(a.out_dir, "emnlp_determinism_report.json")
    with open(path, "w") as f:
        json.dump(report, f, indent=1)
    print(f"wrote {path}; all_equal={all_equal}")
    if not all_equal:
        raise SystemExit("determinism check failed: runs diverged")
    return report


if __name__ == "__main__":
    main()
