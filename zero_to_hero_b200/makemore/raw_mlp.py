"""Character MLP with batch normalisation written on bare tensors: no Module, no optimizer.

What the reference's second makemore script does (nn/makemore/2_1_mlp.py): an embedding table,
one hidden layer `tanh(gain * batchnorm(emb @ W1 + B1) + bias)` and an output layer, trained by
plain SGD on mini-batches; the batch-norm statistics of the training batches are folded by hand
into running estimates (momentum 0.1, biased variance, eps 1e-5, nn/makemore/2_1_mlp.py:110-125)
that replace the batch statistics at evaluation time (nn/makemore/2_1_mlp.py:140-147); the
learning rate is divided once the run passes given fractions of its length
(nn/makemore/2_1_mlp.py:23-24,103-107: the divisor in force is that of the LAST point passed; the
divisors do not multiply).

Here the parameters live in one small state object and the forward pass is a function of
(state, inputs, mode), so the same code serves training, validation and sampling.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F


@dataclass
class RawMLP:
    emb: torch.Tensor          # [vocab, emb_dim]
    w1: torch.Tensor           # [block * emb_dim, hidden]
    b1: torch.Tensor           # [hidden]
    bn_gain: torch.Tensor      # [1, hidden]
    bn_bias: torch.Tensor      # [1, hidden]
    w2: torch.Tensor           # [hidden, vocab]
    b2: torch.Tensor           # [vocab]
    running_mean: torch.Tensor = field(default=None)  # [1, hidden], not trained
    running_var: torch.Tensor = field(default=None)
    momentum: float = 0.1
    eps: float = 1e-5

    def parameters(self) -> list[torch.Tensor]:
        return [self.emb, self.w1, self.b1, self.bn_gain, self.bn_bias, self.w2, self.b2]


def init_raw_mlp(vocab: int, block: int = 4, emb_dim: int = 16, hidden: int = 256,
                 generator: torch.Generator | None = None) -> RawMLP:
    """N(0,1) embeddings; the hidden matrix scaled for tanh with fan-in variance (gain 5/3 over
    sqrt(fan_in)), the output matrix likewise with gain 1; biases zero; batch-norm gain one."""
    g = generator
    fan1 = block * emb_dim
    m = RawMLP(
        emb=torch.randn(vocab, emb_dim, generator=g),
        w1=torch.randn(fan1, hidden, generator=g) * ((5.0 / 3.0) / math.sqrt(fan1)),
        b1=torch.zeros(hidden),
        bn_gain=torch.ones(1, hidden),
        bn_bias=torch.zeros(1, hidden),
        w2=torch.randn(hidden, vocab, generator=g) * (1.0 / math.sqrt(hidden)),
        b2=torch.zeros(vocab),
        running_mean=torch.zeros(1, hidden),
        running_var=torch.ones(1, hidden),
    )
    for p in m.parameters():
        p.requires_grad_(True)
    return m


def forward(m: RawMLP, X: torch.Tensor, train: bool) -> torch.Tensor:
    """Logits [N, vocab] for contexts X [N, block]. In training mode the hidden pre-activations are
    normalised with the statistics of this batch, which are then folded into the running
    estimates; otherwise the running estimates are used and nothing is updated."""
    pre = m.emb[X].flatten(1) @ m.w1 + m.b1
    if train:
        mean = pre.mean(0, keepdim=True)
        var = pre.var(0, keepdim=True, unbiased=False)
        with torch.no_grad():
            m.running_mean.lerp_(mean, m.momentum)
            m.running_var.lerp_(var, m.momentum)
    else:
        mean, var = m.running_mean, m.running_var
    h = torch.tanh(m.bn_gain * (pre - mean) * torch.rsqrt(var + m.eps) + m.bn_bias)
    return h @ m.w2 + m.b2


def step_decay_lr(step: int, steps: int, base: float, points=(0.68, 0.84, 0.92), divisors=(4, 4, 4)) -> float:
    """Base rate divided by the divisor of the last of `points` (fractions of the run) passed."""
    divisor = 1.0
    for frac, d in zip(points, divisors):
        if step >= int(frac * steps):
            divisor = d
    return base / divisor


def train_raw_mlp(m: RawMLP, X: torch.Tensor, Y: torch.Tensor, steps: int, batch_size: int = 256,
                  lr: float = 0.16, generator: torch.Generator | None = None,
                  points=(0.68, 0.84, 0.92), divisors=(4, 4, 4)) -> list[float]:
    """Mini-batch SGD by hand: sample with replacement, forward, clear gradients, backward,
    `p -= lr * grad`. Returns the loss of every step."""
    params = m.parameters()
    history = []
    for step in range(steps):
        rate = step_decay_lr(step, steps, lr, points, divisors)
        idx = torch.randint(0, X.shape[0], (batch_size,), generator=generator)
        loss = F.cross_entropy(forward(m, X[idx], True), Y[idx])
        for p in params:
            p.grad = None
        loss.backward()
        with torch.no_grad():
            for p in params:
                if p.grad is not None:
                    p -= rate * p.grad
        history.append(float(loss.detach()))
    return history


@torch.no_grad()
def evaluate_raw_mlp(m: RawMLP, X: torch.Tensor, Y: torch.Tensor) -> float:
    return float(F.cross_entropy(forward(m, X, False), Y))


@torch.no_grad()
def sample_raw_mlp(m: RawMLP, codec, block: int, n: int, generator: torch.Generator | None = None) -> list[str]:
    out = []
    for _ in range(n):
        ctx, chars = [0] * block, []
        while len(chars) < 40:
            probs = F.softmax(forward(m, torch.tensor([ctx]), False), dim=-1)
            nxt = int(torch.multinomial(probs, 1, generator=generator))
            if nxt == 0:
                break
            chars.append(codec.itos[nxt])
            ctx = ctx[1:] + [nxt]
        out.append("".join(chars))
    return out
