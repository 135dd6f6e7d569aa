"""Datasets, loaders, tokenizer and dataset fetch (crates/data/src/{lib,tokenizer,fetch}.rs, datasets/{sst2,wikitext2}.rs)."""
from .datasets import (Dataset, InMemoryDataset, StreamingDataset, MmapDataset, TokenFileDataset, DataLoaderConfig, DataLoader,
                       simple_loader, shuffled_loader, PinnedBatchPrefetcher, TokenBatchPrefetcher)
from .tokenizer import PAD, UNK, BOS, EOS, Vocab, WordLevelConfig, WordLevelTokenizer
from .fetch import cache_root, fetch_url, FetchError, ungzip, fnv1a64
from .corpora import load_sst2, load_wikitext2, load_wikitext2_splits, Sst2Example, WikiText2Splits

__all__ = [n for n in dir() if not n.startswith("_")]
