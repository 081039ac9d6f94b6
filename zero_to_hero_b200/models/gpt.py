"""Character-level language models: `Vocab`, `BigramLM` and the decoder-only `GPTLM`.

`GPTLM` is the network of the reference's nn/gpt/3_gpt.py:23-149: per-head bias-free
query/key/value projections, scores scaled by head_size**-0.5, causal mask, softmax, dropout
on the attention weights, concatenated heads, output projection, ReLU MLP with two dropouts,
LayerNorm with weight and bias (biased variance, eps 1e-5), pre-norm residual blocks, an
untied head with bias. Parameter names equal the reference's, so its state_dicts load as they
are (its per-head `mask` buffers are not needed and are ignored).

The per-head projections are kept as separate parameters but applied as one fused [3C, C]
matmul followed by the shared causal-attention op, which on a GPU is the flash-attention
kernel when head_size is 64 (6 heads x 384, the benchmark configuration) and dropout is off.
`BigramLM` is nn/gpt/1_bigram.py:22-46: an embedding table read as next-token logits.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as Z
from ..ops.sampling import sample_next


class Vocab:
    """Character codec (nn/gpt/3_gpt.py:9-20)."""

    def __init__(self, text: str):
        self.chars = sorted(set(text))
        self.stoi = {ch: i for i, ch in enumerate(self.chars)}
        self.itos = {i: ch for i, ch in enumerate(self.chars)}
        self.size = len(self.chars)

    def encode(self, seq):
        return [self.stoi[c] for c in seq]

    def decode(self, seq):
        return [self.itos[int(i)] for i in seq]


class Head(nn.Module):
    """Parameter holder for one attention head (applied fused by MultiHeadAttention)."""

    def __init__(self, emb_dim: int, head_size: int):
        super().__init__()
        self.key = nn.Linear(emb_dim, head_size, bias=False)
        self.query = nn.Linear(emb_dim, head_size, bias=False)
        self.value = nn.Linear(emb_dim, head_size, bias=False)


class MultiHeadAttention(nn.Module):
    def __init__(self, block_size: int, emb_dim: int, num_heads: int, dropout: float):
        super().__init__()
        assert emb_dim % num_heads == 0, "emb_dim must be divisible by num_heads"
        self.num_heads = num_heads
        self.heads = nn.ModuleList([Head(emb_dim, emb_dim // num_heads) for _ in range(num_heads)])
        self.proj = nn.Linear(emb_dim, emb_dim)
        self.p = dropout

    def fused_qkv_weight(self) -> torch.Tensor:
        q = torch.cat([h.query.weight for h in self.heads], dim=0)
        k = torch.cat([h.key.weight for h in self.heads], dim=0)
        v = torch.cat([h.value.weight for h in self.heads], dim=0)
        return torch.cat([q, k, v], dim=0)

    def forward(self, X):
        qkv = Z.linear(X, self.fused_qkv_weight())
        o = Z.causal_attention(qkv, self.num_heads, dropout_p=self.p if self.training else 0.0)
        o = Z.linear(o, self.proj.weight, self.proj.bias)
        return F.dropout(o, self.p, self.training)


class FeedForward(nn.Module):
    def __init__(self, emb_dim: int, dropout: float, expansion: int = 4):
        super().__init__()
        self.ff = nn.Sequential(
            nn.Linear(emb_dim, emb_dim * expansion), nn.ReLU(), nn.Dropout(dropout),
            nn.Linear(emb_dim * expansion, emb_dim), nn.Dropout(dropout))

    def forward(self, X):
        h = F.relu(Z.linear(X, self.ff[0].weight, self.ff[0].bias))
        h = self.ff[2](h)
        return self.ff[4](Z.linear(h, self.ff[3].weight, self.ff[3].bias))


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim))

    def forward(self, x):
        return Z.layer_norm(x, self.weight, self.bias, self.eps)


class Block(nn.Module):
    def __init__(self, block_size, emb_dim, num_heads, dropout):
        super().__init__()
        self.ln1 = LayerNorm(emb_dim)
        self.attn = MultiHeadAttention(block_size, emb_dim, num_heads, dropout)
        self.ln2 = LayerNorm(emb_dim)
        self.ff = FeedForward(emb_dim, dropout)

    def forward(self, X):
        X = X + self.attn(self.ln1(X)).to(X.dtype)
        X = X + self.ff(self.ln2(X)).to(X.dtype)
        return X


class GPTLM(nn.Module):
    def __init__(self, vocab_size, block_size, emb_size, num_blocks, num_heads, dropout):
        super().__init__()
        self.block_size = block_size
        self.tok_to_emb = nn.Embedding(vocab_size, emb_size)
        self.pos_to_emb = nn.Embedding(block_size, emb_size)
        self.blocks = nn.Sequential(*[Block(block_size, emb_size, num_heads, dropout)
                                      for _ in range(num_blocks)])
        self.ln = LayerNorm(emb_size)
        self.head = nn.Linear(emb_size, vocab_size)

    def load_reference_state_dict(self, sd: dict[str, torch.Tensor]) -> None:
        self.load_state_dict({k: v for k, v in sd.items() if not k.endswith(".mask")})

    def forward(self, X, Y=None):
        B, T = X.shape
        x = Z.embedding(X, self.tok_to_emb.weight, self.pos_to_emb.weight)
        x = self.blocks(x)
        x = self.ln(x)
        logits = Z.linear(x, self.head.weight, self.head.bias)
        if Y is None:
            return logits, None
        V = logits.shape[-1]
        loss = Z.cross_entropy(logits.reshape(B * T, V), Y.reshape(B * T))
        return logits, loss

    @torch.inference_mode()
    def generate(self, X, max_new_tokens, generator: torch.Generator | None = None):
        """Plain multinomial sampling; crops the context to block_size (the reference feeds the
        whole sequence and so cannot generate past its position table)."""
        for _ in range(max_new_tokens):
            ctx = X if X.size(1) <= self.block_size else X[:, -self.block_size:]
            logits, _ = self(ctx)
            nxt = sample_next(logits[:, -1, :].float(), generator=generator)
            X = torch.cat((X, nxt), dim=1)
        return X


class BigramLM(nn.Module):
    def __init__(self, vocab_size: int):
        super().__init__()
        self.vocab_size = vocab_size
        self.emb = nn.Embedding(vocab_size, vocab_size)

    def forward(self, X, Y=None):
        logits = self.emb(X)
        if Y is None:
            return logits, None
        B, T, C = logits.shape
        return logits, F.cross_entropy(logits.view(B * T, C), Y.view(B * T))

    @torch.inference_mode()
    def generate(self, X, max_new_tokens, generator: torch.Generator | None = None):
        for _ in range(max_new_tokens):
            logits, _ = self(X[:, -1:])
            nxt = sample_next(logits[:, -1, :], generator=generator)
            X = torch.cat((X, nxt), dim=1)
        return X


def causal_average_variants(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Three equivalent ways to average each position with its past (nn/gpt/2_masking.py:13-32):
    explicit loops, a row-normalised lower-triangular matmul, and softmax over a -inf mask."""
    B, T, C = x.shape
    a = torch.zeros_like(x)
    for b in range(B):
        for t in range(T):
            a[b, t] = x[b, : t + 1].mean(0)
    tril = torch.tril(torch.ones(T, T, dtype=x.dtype))
    w = tril / tril.sum(1, keepdim=True)
    b2 = w @ x
    w3 = torch.zeros(T, T, dtype=x.dtype).masked_fill(tril == 0, float("-inf"))
    c = F.softmax(w3, dim=-1) @ x
    return a, b2, c
