"""Token / label vocabulary (crates/symbolic/src/lib.rs)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class LabelPrediction:
    label: str
    id: int
    score: float


class SymbolicError(ValueError):
    """crates/symbolic/src/lib.rs:10-18: an insert into a frozen vocabulary (`kind` "frozen") or an id outside it
    (`kind` "id_out_of_range"); raised by the strict accessors `try_insert` and `token_strict`."""

    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


class Vocabulary:
    """Insert-ordered symbol table with an unknown token at id 0; `freeze()` stops growth."""

    def __init__(self, unk: str = "<unk>"):
        self._tokens: list = []
        self._ids: dict = {}
        self._frozen = False
        self.unk = unk
        self.insert(unk)

    @classmethod
    def with_specials(cls, unk: str = "<unk>", specials=()) -> "Vocabulary":
        v = cls(unk)
        for s in specials:
            v.insert(s)
        return v

    def insert(self, token: str) -> int:
        i = self._ids.get(token)
        if i is not None:
            return i
        if self._frozen:
            return self._ids[self.unk]
        i = len(self._tokens)
        self._tokens.append(token)
        self._ids[token] = i
        return i

    def try_insert(self, token: str) -> int:
        """`insert` that refuses a new token once the vocabulary is frozen instead of mapping it to the unknown id."""
        if self._frozen and token not in self._ids:
            raise SymbolicError("frozen", f"vocabulary is frozen; cannot insert token {token!r}")
        return self.insert(token)

    def token_strict(self, i: int) -> str:
        if not (0 <= i < len(self._tokens)):
            raise SymbolicError("id_out_of_range", f"id {i} is out of range")
        return self._tokens[i]

    def freeze(self) -> None:
        self._frozen = True

    def is_frozen(self) -> bool:
        return self._frozen

    def id(self, token: str):
        return self._ids.get(token)

    def id_or_unk(self, token: str) -> int:
        return self._ids.get(token, self._ids[self.unk])

    def token(self, i: int):
        return self._tokens[i] if 0 <= i < len(self._tokens) else None

    def tokens(self) -> list:
        return list(self._tokens)

    def __len__(self):
        return len(self._tokens)

    def __contains__(self, token):
        return token in self._ids
