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
        ctx = list(ex["ctx_tokens"])
        label = int(ex["label"])
        t = torch.zeros(4, MAX_LEN, dtype=torch.long)
        mask = torch.zeros(4, MAX_LEN)
        for j, end in enumerate(ex["ending_tokens"]):
            toks = (ctx + list(end))[-block_size:][:MAX_LEN]
            start = len(toks) - len(end)
            t[j, :len(toks)] = torch.tensor(toks)
            mask[j, start:len(toks)] = 1.0
        t, mask = t.to(device), mask.to(device)
        logits = logits_fn(t).float()
        # position p predicts token p+1
        ce = F.cross_entropy(logits[:, :-1].reshape(-1, logits.size(-1)), t[:, 1:].reshape(-1),
                             reduction="none").view(4, -1)
        m = mask[:, 1:]
        losses = (ce * m).sum(1) / m.sum(1).clamp_min(1.0)
        correct += int(int(losses.argmin()) == label)
        total += 1
    return correct, total
