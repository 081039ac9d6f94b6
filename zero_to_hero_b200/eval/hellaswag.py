"""HellaSwag multiple-choice evaluation, offline.

Same scoring as the reference (nn/gpt2/hellaswag.py:21-62): each example's four
context+ending sequences are padded to a fixed (4, 256) batch, one forward gives logits at
all positions, an ending's score is the mean cross-entropy over its tokens, the prediction is
the argmin; examples are strided across ranks and the caller sums `correct`/`total` over ranks.
Differences: examples are read from a local JSONL file whose rows already hold token ids
(`{"ctx_tokens": [...], "ending_tokens": [[...] x4], "label": k}`) because neither the
dataset nor the BPE tables can be downloaded here, and the per-ending losses are reduced on
the device (one host sync per example instead of four).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch
import torch.nn.functional as F

MAX_LEN = 256


def load_examples(path: str | Path) -> list[dict]:
    return [json.loads(line) for line in Path(path).read_text().splitlines() if line.strip()]


def example_tensors(ex: dict, block_size: int):
    """One example as the reference batches it (nn/gpt2/hellaswag.py:30-44): tokens [4, 256]
    (context + ending, zero padded), a mask over the ending's positions, and the label."""
    ctx = list(ex["ctx_tokens"])
    t = torch.zeros(4, MAX_LEN, dtype=torch.long)
    mask = torch.zeros(4, MAX_LEN)
    for j, end in enumerate(ex["ending_tokens"]):
        toks = (ctx + list(end))[-block_size:][:MAX_LEN]
        start = len(toks) - len(end)
        t[j, :len(toks)] = torch.tensor(toks)
        mask[j, start:len(toks)] = 1.0
    return t, mask, int(ex["label"])


def _score(ce: torch.Tensor, mask: torch.Tensor) -> int:
    """ce[4, 255]: loss of predicting token p+1 at position p. Returns the argmin ending."""
    m = mask[:, 1:]
    losses = (ce * m).sum(1) / m.sum(1).clamp_min(1.0)
    return int(losses.argmin())


@torch.inference_mode()
def evaluate(model, examples: list[dict], device, block_size: int, rank: int = 0, world_size: int = 1,
             logits_fn=None):
    """Returns (correct, total) tensors on `device`. `logits_fn(tokens[4, T]) -> logits[4, T, V]`
    defaults to `model(tokens, dummy_targets)[0]`."""
    correct = torch.tensor(0, device=device)
    total = torch.tensor(0, device=device)
    if logits_fn is None:
        def logits_fn(t):
            return model(t, torch.zeros_like(t))[0]
    for i, ex in enumerate(examples):
        if i % world_size != rank:
            continue
        t, mask, label = example_tensors(ex, block_size)
        t, mask = t.to(device), mask.to(device)
        logits = logits_fn(t).float()
        # position p predicts token p+1
        ce = F.cross_entropy(logits[:, :-1].reshape(-1, logits.size(-1)), t[:, 1:].reshape(-1),
                             reduction="none").view(4, -1)
        correct += int(_score(ce, mask) == label)
        total += 1
    return correct, total


@torch.inference_mode()
def evaluate_losses_fn(losses_fn, examples: list[dict], device, block_size: int, rank: int = 0,
                       world_size: int = 1):
    """Same scoring when the model hands back per-token losses instead of logits:
    `losses_fn(tokens[4, 256], targets[4, 256]) -> loss[4, 256]` with targets = tokens shifted
    left by one. This is the route through the fused engine's forward-only pass, which never
    moves the (4, 256, V) logits out of its own buffers."""
    correct = torch.tensor(0, device=device)
    total = torch.tensor(0, device=device)
    for i, ex in enumerate(examples):
        if i % world_size != rank:
            continue
        t, mask, label = example_tensors(ex, block_size)
        tgt = torch.zeros_like(t)
        tgt[:, :-1] = t[:, 1:]
        ce = losses_fn(t, tgt)[:, :-1].float()
        correct += int(_score(ce, mask.to(ce.device)) == label)
        total += 1
    return correct, total
