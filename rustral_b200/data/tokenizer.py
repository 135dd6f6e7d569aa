"""Word-level tokenizer (crates/data/src/tokenizer.rs): specials PAD=0, UNK=1, BOS=2, EOS=3; vocabulary ordered by
descending frequency with lexicographic ties."""
from __future__ import annotations

from collections import Counter
from dataclasses import dataclass

PAD, UNK, BOS, EOS = "<pad>", "<unk>", "<bos>", "<eos>"


class Vocab:
    def __init__(self, tokens):
        self.tokens = list(tokens)
        self.id_of = {t: i for i, t in enumerate(self.tokens)}
        self.pad_id, self.unk_id, self.bos_id, self.eos_id = (self.id_of[s] for s in (PAD, UNK, BOS, EOS))

    def __len__(self):
        return len(self.tokens)


@dataclass
class WordLevelConfig:
    lowercase: bool = True
    max_vocab: int = 0          # 0 = unlimited (specials included in the count)
    min_freq: int = 1


class WordLevelTokenizer:
    def __init__(self, vocab: Vocab, config: WordLevelConfig | None = None):
        self.vocab, self.config = vocab, config or WordLevelConfig()

    def _split(self, text: str) -> list:
        return (text.lower() if self.config.lowercase else text).split()

    @classmethod
    def fit_from_iter(cls, texts, config: WordLevelConfig | None = None) -> "WordLevelTokenizer":
        config = config or WordLevelConfig()
        tmp = cls(Vocab([PAD, UNK, BOS, EOS]), config)
        counts = Counter()
        for t in texts:
            counts.update(tmp._split(t))
        words = sorted((w for w, c in counts.items() if c >= config.min_freq and w not in (PAD, UNK, BOS, EOS)),
                       key=lambda w: (-counts[w], w))
        if config.max_vocab > 0:
            words = words[:max(0, config.max_vocab - 4)]
        return cls(Vocab([PAD, UNK, BOS, EOS] + words), config)

    @classmethod
    def from_vocab_file(cls, path: str, config: WordLevelConfig | None = None) -> "WordLevelTokenizer":
        with open(path, encoding="utf-8") as f:
            toks = [l.rstrip("\n") for l in f if l.strip()]
        for i, s in enumerate((PAD, UNK, BOS, EOS)):
            if len(toks) <= i or toks[i] != s:
                raise ValueError(f"vocabulary file must start with the specials; line {i + 1} should be {s}")
        return cls(Vocab(toks), config)

    def save_vocab(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as f:
            f.write("\n".join(self.vocab.tokens) + "\n")

    def encode(self, text: str) -> list:
        v = self.vocab
        return [v.id_of.get(w, v.unk_id) for w in self._split(text)]

    def encode_with_specials(self, text: str) -> list:
        return [self.vocab.bos_id] + self.encode(text) + [self.vocab.eos_id]

    def decode(self, ids) -> str:
        v = self.vocab
        skip = {v.pad_id, v.bos_id, v.eos_id}
        return " ".join(v.tokens[i] if 0 <= i < len(v) else UNK for i in ids if i not in skip)
