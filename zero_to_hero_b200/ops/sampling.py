"""Next-token sampling: temperature, top-k, softmax, multinomial
(nn/gpt2/modules.py:130-135; the char-level models sample without temperature/top-k,
nn/gpt/3_gpt.py:141-149)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def sample_next(logits: torch.Tensor, temperature: float = 1.0, top_k: int | None = None,
                generator: torch.Generator | None = None) -> torch.Tensor:
    """logits [B, V] -> sampled ids [B, 1]."""
    logits = logits / temperature
    if top_k is not None:
        v, _ = torch.topk(logits, min(top_k, logits.size(-1)))
        logits = logits.masked_fill(logits < v[:, [-1]], -float("inf"))
    probs = F.softmax(logits, dim=-1)
    return torch.multinomial(probs, num_samples=1, generator=generator)
