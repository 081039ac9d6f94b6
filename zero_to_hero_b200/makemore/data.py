"""Names data: loading, a '.'-delimited character codec, context-window datasets.

The reference reads nn/makemore/names.txt (32,032 names) next to its scripts; here the path is
an argument (default: the installed copy of the reference data if present) and
`synthetic_names` produces a seeded stand-in corpus so tests and demos run without the file.
"""
from __future__ import annotations

import random
from pathlib import Path

import torch

_DEFAULT = Path(__file__).resolve().parents[2] / "baseline" / "_ref" / "nn" / "makemore" / "names.txt"


def load_names(path: str | Path | None = None) -> list[str]:
    p = Path(path) if path else _DEFAULT
    if not p.exists():
        raise FileNotFoundError(f"{p} not found; pass a names file or use synthetic_names()")
    return p.read_text().splitlines()


def synthetic_names(n: int = 2000, seed: int = 0) -> list[str]:
    """Pronounceable pseudo-names from a small syllable grammar (deterministic per seed)."""
    rng = random.Random(seed)
    onsets = ["", "b", "c", "d", "j", "k", "l", "m", "n", "r", "s", "t", "v", "z", "br", "ch", "sh", "th"]
    vowels = ["a", "e", "i", "o", "u", "ia", "ee", "ay", "y"]
    codas = ["", "", "n", "l", "r", "s", "h", "m"]
    out = []
    for _ in range(n):
        k = rng.choice([1, 2, 2, 3])
        name = "".join(rng.choice(onsets) + rng.choice(vowels) + rng.choice(codas) for _ in range(k))
        out.append(name[:12] or "a")
    return out


class CharCodec:
    """Characters of the corpus plus '.', the boundary token with id 0."""

    def __init__(self, names: list[str]):
        self.chars = sorted(set("".join(names) + "."))
        self.stoi = {c: i for i, c in enumerate(self.chars)}
        self.itos = {i: c for c, i in self.stoi.items()}
        assert self.stoi["."] == 0

    @property
    def size(self) -> int:
        return len(self.chars)

    def decode(self, ids) -> str:
        return "".join(self.itos[int(i)] for i in ids)


def build_dataset(names: list[str], codec: CharCodec, block_size: int) -> tuple[torch.Tensor, torch.Tensor]:
    """X[i] = the `block_size` characters before position i (padded with '.'), Y[i] = the next."""
    X, Y = [], []
    for name in names:
        ctx = [0] * block_size
        for ch in name + ".":
            ix = codec.stoi[ch]
            X.append(ctx)
            Y.append(ix)
            ctx = ctx[1:] + [ix]
    return torch.tensor(X), torch.tensor(Y)


def split_names(names: list[str], seed: int = 42, fractions=(0.8, 0.1)) -> tuple[list, list, list]:
    names = list(names)
    random.Random(seed).shuffle(names)
    n1 = int(fractions[0] * len(names))
    n2 = int((fractions[0] + fractions[1]) * len(names))
    return names[:n1], names[n1:n2], names[n2:]
