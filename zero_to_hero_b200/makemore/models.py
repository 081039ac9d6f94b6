"""MLP and WaveNet-style name models on the hand-rolled layers, with their training loop
(nn/makemore/2_1_mlp.py, 2_2_mlp_modularlized.py:157-283, 4_1_wavenet.py:229-298)."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .layers import BatchNorm1d, Embedding, Flatten, FlattenConsecutive, Linear, Sequential, Tanh


def build_mlp(vocab: int, block_size: int = 4, emb: int = 16, hidden: int = 256, depth: int = 4, generator=None):
    """Embedding -> Flatten -> depth x (Linear, BatchNorm, Tanh) -> Linear; the output layer is
    scaled down so the initial loss is near log(vocab)."""
    layers = [Embedding(vocab, emb, generator), Flatten()]
    fan_in = emb * block_size
    for _ in range(depth):
        layers += [Linear(fan_in, hidden, bias=False, generator=generator), BatchNorm1d(hidden), Tanh()]
        fan_in = hidden
    out = Linear(fan_in, vocab, generator=generator)
    with torch.no_grad():
        out.weight *= 0.1
    return Sequential(*layers, out)


def build_wavenet(vocab: int, block_size: int = 8, emb: int = 24, hidden: int = 128, generator=None):
    """log2(block_size) stages that each merge neighbouring pairs of positions."""
    stages = int(math.log2(block_size))
    assert 2 ** stages == block_size, "block_size must be a power of two"
    layers = [Embedding(vocab, emb, generator)]
    fan_in = emb
    for _ in range(stages):
        layers += [FlattenConsecutive(2), Linear(fan_in * 2, hidden, bias=False, generator=generator),
                   BatchNorm1d(hidden), Tanh()]
        fan_in = hidden
    out = Linear(hidden, vocab, generator=generator)
    with torch.no_grad():
        out.weight *= 0.1
    return Sequential(*layers, out)


def train_model(model, X, Y, steps: int = 1000, batch_size: int = 32, lr: float = 0.1, decay_at: float = 0.75,
                generator=None) -> list[float]:
    """Minibatch SGD with a 10x step decay after `decay_at` of the steps."""
    model.train()
    losses = []
    params = model.parameters()
    for step in range(steps):
        ix = torch.randint(0, X.shape[0], (batch_size,), generator=generator)
        loss = F.cross_entropy(model(X[ix]), Y[ix])
        for p in params:
            p.grad = None
        loss.backward()
        cur = lr if step < decay_at * steps else lr / 10
        with torch.no_grad():
            for p in params:
                p -= cur * p.grad
        losses.append(loss.item())
    return losses


@torch.no_grad()
def evaluate(model, X, Y) -> float:
    model.eval()
    loss = F.cross_entropy(model(X), Y).item()
    model.train()
    return loss


@torch.no_grad()
def sample(model, codec, block_size: int, n: int = 8, generator=None) -> list[str]:
    model.eval()
    out = []
    for _ in range(n):
        ctx, chars = [0] * block_size, []
        while len(chars) < 40:
            probs = F.softmax(model(torch.tensor([ctx])), dim=-1).reshape(-1)
            ix = int(torch.multinomial(probs, 1, generator=generator).item())
            if ix == 0:
                break
            chars.append(codec.itos[ix])
            ctx = ctx[1:] + [ix]
        out.append("".join(chars))
    model.train()
    return out
