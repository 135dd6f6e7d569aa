"""SST-2 and WikiText-2 loaders (crates/data/src/datasets/sst2.rs:56, wikitext2.rs:42).

Files are taken from the cache (`<cache>/datasets/sst2/{train,dev}.jsonl`, `<cache>/datasets/wikitext-2/wiki.{train,valid,test}.tokens`);
when absent and not offline they are downloaded from the URLs below.  Tests stage tiny synthetic corpora into a
temporary RUSTRAL_CACHE_DIR with RUSTRAL_DATASET_OFFLINE=1, as the reference's smoke tests do."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

from .fetch import cache_root, fetch_url

SST2_URLS = {"train": "https://huggingface.co/datasets/SetFit/sst2/resolve/main/train.jsonl",
             "dev": "https://huggingface.co/datasets/SetFit/sst2/resolve/main/dev.jsonl"}
WIKITEXT2_URLS = {s: f"https://huggingface.co/datasets/wikitext/resolve/main/wikitext-2-raw-v1/wiki.{s}.tokens"
                  for s in ("train", "valid", "test")}


@dataclass
class Sst2Example:
    text: str
    label: int


def _parse_sst2_tsv(path: str) -> list:
    """`sentence<TAB>label` lines under a header row (the legacy GLUE layout, sst2.rs:93)."""
    out = []
    with open(path, encoding="utf-8") as f:
        for i, line in enumerate(f):
            line = line.rstrip("\n")
            if not line or (i == 0 and line.lower().startswith("sentence")):
                continue
            text, _, label = line.rpartition("\t")
            if text and label.strip() in ("0", "1"):
                out.append(Sst2Example(text, int(label)))
    return out


def load_sst2(split: str = "train") -> list:
    name = {"train": "train.jsonl", "dev": "dev.jsonl", "validation": "dev.jsonl"}[split]
    path = os.path.join(cache_root(), "datasets", "sst2", name)
    legacy = path[:-len(".jsonl")] + ".tsv"
    if not os.path.exists(path) and os.path.exists(legacy):
        return _parse_sst2_tsv(legacy)
    if not os.path.exists(path):
        path = fetch_url(SST2_URLS["train" if split == "train" else "dev"], None, os.path.join("datasets", "sst2"), name)
    out = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line:
                r = json.loads(line)
                out.append(Sst2Example(r["text"], int(r["label"])))
    return out


@dataclass
class WikiText2Splits:
    """The three splits as text (crates/data/src/datasets/wikitext2.rs:31-35)."""
    train: str
    valid: str
    test: str

    def __iter__(self):
        return iter((self.train, self.valid, self.test))


def load_wikitext2_splits() -> WikiText2Splits:
    """All three splits at once, each from the cache or fetched like `load_wikitext2(split)`."""
    return WikiText2Splits(load_wikitext2("train"), load_wikitext2("valid"), load_wikitext2("test"))


def load_wikitext2(split: str = "train") -> str:
    name = f"wiki.{split}.tokens"
    path = os.path.join(cache_root(), "datasets", "wikitext-2", name)
    legacy = os.path.join(cache_root(), "datasets", "wikitext-2", f"{split}.txt")     # pre-staged plain-text layout
    if not os.path.exists(path) and os.path.exists(legacy):
        path = legacy
    if not os.path.exists(path):
        path = fetch_url(WIKITEXT2_URLS[split], None, os.path.join("datasets", "wikitext-2"), name)
    with open(path, encoding="utf-8") as f:
        return f.read()
