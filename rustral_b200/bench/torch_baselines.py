"""Plain-PyTorch comparison baselines for the two NLP tasks (benchmarks/pytorch/sst2_baseline.py,
benchmarks/pytorch/wikitext2_baseline.py): the same data, tokenizer, model shape and optimizer as the examples, but
built from `torch.nn` modules and `torch.optim.Adam` with no code of this framework on the training path.  Each run
writes a manifest with `"framework": "pytorch"`; several seeds are curated into `<task>_pytorch.json`, the file the
comparison reports put next to the framework's own `<task>.json`.

    python -m rustral_b200.bench.torch_baselines --task sst2 --seeds 0,1,2 --vocab out/sst2/vocab.txt --out runs/nlp
    python -m rustral_b200.bench.torch_baselines --task wikitext2 --quick
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..data.corpora import load_sst2, load_wikitext2
from ..data.fetch import fnv1a64
from ..data.tokenizer import WordLevelConfig, WordLevelTokenizer
from .manifest import curate, detect_git_sha, validate_curated


class _Encoder(nn.Module):
    """Token + learned positional embedding, pre-LN transformer layers (GELU), final LayerNorm."""

    def __init__(self, vocab, seq_len, d_model, heads, ffn, layers):
        super().__init__()
        self.tok, self.pos = nn.Embedding(vocab, d_model), nn.Embedding(seq_len, d_model)
        layer = nn.TransformerEncoderLayer(d_model, heads, ffn, dropout=0.0, activation="gelu", batch_first=True, norm_first=True)
        self.layers = nn.TransformerEncoder(layer, layers, enable_nested_tensor=False)
        self.norm = nn.LayerNorm(d_model)
        for p in (self.tok.weight, self.pos.weight):
            nn.init.normal_(p, std=0.02)

    def forward(self, ids, causal=False, pad_mask=None):
        S = ids.shape[1]
        x = self.tok(ids) + self.pos(torch.arange(S, device=ids.device))[None]
        mask = torch.triu(torch.full((S, S), float("-inf"), device=ids.device), 1) if causal else None
        return self.norm(self.layers(x, mask=mask, src_key_padding_mask=pad_mask))


class Sst2Torch(nn.Module):
    def __init__(self, vocab, seq_len, d_model, heads, ffn, layers, pad_id=0):
        super().__init__()
        self.enc, self.head, self.pad_id = _Encoder(vocab, seq_len, d_model, heads, ffn, layers), nn.Linear(d_model, 2), pad_id

    def forward(self, ids):
        keep = (ids != self.pad_id).float()
        h = self.enc(ids)
        pooled = (h * keep[..., None]).sum(1) / keep.sum(1, keepdim=True).clamp_min(1.0)
        return self.head(pooled)


class WordLMTorch(nn.Module):
    def __init__(self, vocab, block, d_model, heads, ffn, layers):
        super().__init__()
        self.enc, self.head = _Encoder(vocab, block, d_model, heads, ffn, layers), nn.Linear(d_model, vocab, bias=False)

    def forward(self, ids):
        return self.head(self.enc(ids, causal=True))


def _batches(n, batch, seed, epoch):
    g = torch.Generator().manual_seed(seed * 1000003 + epoch)
    perm = torch.randperm(n, generator=g)
    return [perm[i:i + batch] for i in range(0, n, batch)]


def run_sst2(a, seed: int) -> dict:
    torch.manual_seed(seed)
    train, dev = load_sst2("train"), load_sst2("dev")
    if a.quick:
        train, dev = train[:256], dev[:256]
    tok = (WordLevelTokenizer.from_vocab_file(a.vocab) if a.vocab else
           WordLevelTokenizer.fit_from_iter((e.text for e in train), WordLevelConfig(lowercase=True, max_vocab=8192)))

    def enc(rows):
        ids = [(tok.encode(e.text)[:a.seq_len] + [tok.vocab.pad_id] * a.seq_len)[:a.seq_len] for e in rows]
        return torch.tensor(ids), torch.tensor([e.label for e in rows])
    (xt, yt), (xd, yd) = enc(train), enc(dev)
    dev_ = torch.device(a.device)
    model = Sst2Torch(len(tok.vocab), a.seq_len, a.d_model, a.num_heads, a.ffn_dim, a.num_layers, tok.vocab.pad_id).to(dev_)
    opt = torch.optim.Adam(model.parameters(), lr=a.lr)
    t0, losses = time.perf_counter(), []
    for ep in range(a.epochs):
        tot = 0.0
        for idx in _batches(len(xt), a.batch_size, seed, ep):
            loss = F.cross_entropy(model(xt[idx].to(dev_)), yt[idx].to(dev_))
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
            tot += float(loss.detach()) * len(idx)
        losses.append(tot / len(xt))
    elapsed = time.perf_counter() - t0
    model.eval()
    with torch.no_grad():
        logits = torch.cat([model(xd[i:i + 256].to(dev_)).float().cpu() for i in range(0, len(xd), 256)])
    digest = fnv1a64("\n".join(f"{e.label}\t{e.text}" for e in train + dev).encode("utf-8"))
    return {"task": "sst2_classifier", "framework": "pytorch", "torch_version": torch.__version__, "model_type": "transformer_encoder",
            "git_sha": detect_git_sha(), "seed": seed, "seq_len": a.seq_len, "d_model": a.d_model, "num_heads": a.num_heads,
            "ffn_dim": a.ffn_dim, "num_layers": a.num_layers, "total_params": sum(p.numel() for p in model.parameters()),
            "vocab_size": len(tok.vocab), "epochs": a.epochs, "batch_size": a.batch_size, "learning_rate": a.lr,
            "train_examples": len(train), "dev_examples": len(dev), "dataset_hash_fnv1a": f"{digest:016x}",
            "dev_loss": float(F.cross_entropy(logits, yd)), "dev_accuracy": float((logits.argmax(-1) == yd).float().mean()),
            "samples_per_sec": a.epochs * len(xt) / max(elapsed, 1e-9), "train_elapsed_sec": elapsed, "epoch_losses": losses,
            "dataset": "SST-2 (binary, HuggingFace SetFit/sst2 mirror)", "tokenizer": "WordLevelTokenizer (whitespace, lowercased)",
            "device": str(dev_), "quick_mode": bool(a.quick)}


def run_wikitext2(a, seed: int) -> dict:
    torch.manual_seed(seed)
    train_text, valid_text = load_wikitext2("train"), load_wikitext2("valid")
    tok = WordLevelTokenizer.fit_from_iter([train_text], WordLevelConfig(lowercase=True, max_vocab=16384))
    cap = 4000 if a.quick else a.train_tokens
    block = a.seq_len

    def windows(text):
        ids = tok.encode(text)[:cap or None]
        n = (len(ids) - 1) // block
        x = torch.tensor(ids[:n * block]).view(n, block)
        y = torch.tensor(ids[1:n * block + 1]).view(n, block)
        return x, y
    (xt, yt), (xv, yv) = windows(train_text), windows(valid_text)
    if not len(xt) or not len(xv):
        raise SystemExit(f"corpus too small for block size {block}")
    dev_ = torch.device(a.device)
    model = WordLMTorch(len(tok.vocab), block, a.d_model, a.num_heads, a.ffn_dim, a.num_layers).to(dev_)
    opt = torch.optim.Adam(model.parameters(), lr=a.lr)
    t0, losses = time.perf_counter(), []
    for ep in range(a.epochs):
        tot = 0.0
        for idx in _batches(len(xt), a.batch_size, seed, ep):
            logits = model(xt[idx].to(dev_))
            loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), yt[idx].to(dev_).reshape(-1))
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
            tot += float(loss.detach()) * len(idx)
        losses.append(tot / len(xt))
    elapsed = time.perf_counter() - t0
    model.eval()
    with torch.no_grad():
        tot, n = 0.0, 0
        for i in range(0, len(xv), 64):
            lg = model(xv[i:i + 64].to(dev_)).float().cpu()
            tot += float(F.cross_entropy(lg.reshape(-1, lg.shape[-1]), yv[i:i + 64].reshape(-1), reduction="sum"))
            n += yv[i:i + 64].numel()
    val = tot / max(1, n)
    digest = fnv1a64((train_text + "\n" + valid_text).encode("utf-8"))
    return {"task": "wikitext2_word_lm", "framework": "pytorch", "torch_version": torch.__version__, "model_type": "transformer_lm",
            "git_sha": detect_git_sha(), "seed": seed, "block_size": block, "d_model": a.d_model, "num_heads": a.num_heads,
            "ffn_dim": a.ffn_dim, "num_layers": a.num_layers, "total_params": sum(p.numel() for p in model.parameters()),
            "vocab_size": len(tok.vocab), "epochs": a.epochs, "batch_size": a.batch_size, "learning_rate": a.lr,
            "train_windows": len(xt), "valid_windows": len(xv), "dataset_hash_fnv1a": f"{digest:016x}",
            "dev_loss_nats": val, "dev_perplexity": math.exp(min(val, 50.0)),
            "windows_per_sec": a.epochs * len(xt) / max(elapsed, 1e-9), "train_elapsed_sec": elapsed, "epoch_losses": losses,
            "dataset": "WikiText-2 raw v1", "tokenizer": "WordLevelTokenizer (whitespace, lowercased)", "device": str(dev_),
            "quick_mode": bool(a.quick)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="rustral_b200.bench.torch_baselines", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--task", choices=["sst2", "wikitext2"], required=True)
    ap.add_argument("--seeds", default="0,1,2")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--vocab", help="(sst2) vocab.txt written by examples/sst2_classifier.py, for identical token ids")
    ap.add_argument("--seq-len", type=int, default=32, help="sequence length (sst2) / block size (wikitext2)")
    ap.add_argument("--d-model", type=int, default=64)
    ap.add_argument("--num-heads", type=int, default=4)
    ap.add_argument("--ffn-dim", type=int, default=128)
    ap.add_argument("--num-layers", type=int, default=2)
    ap.add_argument("--lr", type=float, default=5e-4)
    ap.add_argument("--batch-size", type=int, default=32)
    ap.add_argument("--epochs", type=int, default=0, help="0 = the example's default (3 for sst2, 1 for wikitext2)")
    ap.add_argument("--train-tokens", type=int, default=50000)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--out", default=os.path.join("benchmarks", "runs", "v0.1.0", "nlp"))
    a = ap.parse_args(argv)
    a.epochs = a.epochs or (1 if (a.quick or a.task == "wikitext2") else 3)
    run = run_sst2 if a.task == "sst2" else run_wikitext2
    metric = "dev_accuracy" if a.task == "sst2" else "dev_perplexity"
    manifests = [run(a, int(s)) for s in a.seeds.split(",") if s.strip()]
    doc = curate(manifests[0]["task"], metric, os.environ.get("RUSTRAL_EVAL_VERSION", "0.1.0"), manifests)
    problems = validate_curated(doc)
    if problems:
        raise SystemExit("\n".join(problems))
    os.makedirs(a.out, exist_ok=True)
    path = os.path.join(a.out, f"{a.task}_pytorch.json")
    with open(path, "w", encoding="utf-8") as f:
        json.dump(doc, f, indent=2)
        f.write("\n")
    agg = doc["aggregate"]
    print(f"{a.task} (pytorch): {metric} mean={agg['mean']:.4f} std={agg['std']:.4f} over {agg['n']} seed(s) -> {path}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
