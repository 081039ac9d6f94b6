"""Bigram name models three ways (nn/makemore/1_1_bigram_stat.py, 1_2_bigram_nn_micrograd.py,
1_3_bigram_nn_torch.py of the reference): a count table with add-one smoothing, a one-layer
softmax network on one-hot inputs trained with plain gradient descent in PyTorch, and the same
network built from micrograd `Value`s."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .data import CharCodec


def bigram_pairs(names, codec: CharCodec) -> tuple[torch.Tensor, torch.Tensor]:
    xs, ys = [], []
    for name in names:
        chs = ["."] + list(name) + ["."]
        for a, b in zip(chs, chs[1:]):
            xs.append(codec.stoi[a])
            ys.append(codec.stoi[b])
    return torch.tensor(xs), torch.tensor(ys)


def bigram_counts(names, codec: CharCodec) -> torch.Tensor:
    xs, ys = bigram_pairs(names, codec)
    counts = torch.zeros(codec.size, codec.size, dtype=torch.int32)
    counts.index_put_((xs, ys), torch.ones_like(xs, dtype=torch.int32), accumulate=True)
    return counts


def bigram_probs(counts: torch.Tensor, smoothing: int = 0) -> torch.Tensor:
    """Row-normalised counts; with smoothing k the reference divides by (row sum + V) after adding
    k to every cell (1_1_bigram_stat.py:66-69)."""
    c = (counts + smoothing).float()
    denom = c.sum(dim=1, keepdim=True) + (counts.shape[0] if smoothing else 0)
    return c / denom


def sample_names(probs: torch.Tensor, codec: CharCodec, n: int, generator=None) -> list[str]:
    out = []
    for _ in range(n):
        ix, chars = 0, []
        while True:
            ix = int(torch.multinomial(probs[ix], 1, generator=generator).item())
            if ix == 0:
                break
            chars.append(codec.itos[ix])
        out.append("".join(chars))
    return out


def average_nll(names, probs: torch.Tensor, codec: CharCodec) -> float:
    xs, ys = bigram_pairs(names, codec)
    return float(-probs[xs, ys].log().mean())


def train_bigram_torch(names, codec: CharCodec, epochs: int = 256, lr: float = 64.0, seed: int = 42):
    """logits = onehot(x) @ W, full-batch gradient descent; returns (W, loss history)."""
    xs, ys = bigram_pairs(names, codec)
    g = torch.Generator().manual_seed(seed)
    W = torch.randn(codec.size, codec.size, generator=g, requires_grad=True)
    xenc = F.one_hot(xs, codec.size).float()
    losses = []
    for _ in range(epochs):
        loss = F.cross_entropy(xenc @ W, ys)
        losses.append(loss.item())
        W.grad = None
        loss.backward()
        W.data -= lr * W.grad
    return W.detach(), losses


def train_bigram_micrograd(names, codec: CharCodec, epochs: int = 10, lr: float = 1.0, seed: int = 42):
    """The same model with scalar `Value`s (slow by construction: use a handful of names)."""
    import random

    from ..micrograd import Value

    xs, ys = bigram_pairs(names, codec)
    rng = random.Random(seed)
    V = codec.size
    W = [[Value(rng.gauss(0, 1)) for _ in range(V)] for _ in range(V)]
    losses = []
    for _ in range(epochs):
        total = Value(0.0)
        for x, y in zip(xs.tolist(), ys.tolist()):
            exps = [w.exp() for w in W[x]]  # one-hot @ W selects row x
            denom = sum(exps[1:], exps[0])
            total = total + (-(exps[y] / denom).log())
        loss = total * (1.0 / len(xs))
        losses.append(loss.data)
        for row in W:
            for w in row:
                w.grad = 0.0
        loss.backward()
        for row in W:
            for w in row:
                w.data -= lr * w.grad
    return W, losses
