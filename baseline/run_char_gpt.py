"""Char-level GPT on CPU, fp32, single process: the benchmark's first configuration, both arms.

    python baseline/run_char_gpt.py --impl ours        # zero_to_hero_b200.models.gpt.GPTLM
    python baseline/run_char_gpt.py --impl reference   # the unmodified nn/gpt/3_gpt.py classes

6 layers, 6 heads, width 384, context 256, vocabulary 65, dropout 0.2, batch 64, AdamW lr 3e-4,
20 training steps on seeded uniform tokens (targets = inputs shifted by one), then 100 sampled
tokens. The reference script itself hard-codes another shape and reads a text file
(nn/gpt/3_gpt.py:153-202), but its classes take every size as an argument (nn/gpt/3_gpt.py:109-111),
so they are imported unchanged from the installed copy of the reference and driven with the
same loop (forward, zero_grad, backward, step: nn/gpt/3_gpt.py:226-232). Prints one JSON line.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
V, T, C, L, H, DROPOUT, B, LR, STEPS, NEW_TOKENS = 65, 256, 384, 6, 6, 0.2, 64, 3e-4, 20, 100


def build(impl: str):
    if impl == "ours":
        from zero_to_hero_b200.models.gpt import GPTLM
        return GPTLM(V, T, C, L, H, DROPOUT)
    path = ROOT / "baseline" / "_ref" / "nn" / "gpt" / "3_gpt.py"
    if not path.exists():
        raise SystemExit(json.dumps({"impl": "reference", "unavailable": f"{path} is missing"}))
    spec = importlib.util.spec_from_file_location("z2h_reference_char_gpt", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.GPTLM(V, T, C, L, H, DROPOUT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--steps", type=int, default=STEPS)
    ap.add_argument("--threads", type=int, default=0)
    a = ap.parse_args()
    if a.threads:
        torch.set_num_threads(a.threads)
    torch.manual_seed(42)
    model = build(a.impl)
    n_params = sum(p.numel() for p in model.parameters())
    opt = torch.optim.AdamW(model.parameters(), lr=LR)
    g = torch.Generator().manual_seed(1234)
    model.train()
    losses = []
    t0 = time.perf_counter()
    for _ in range(a.steps):
        tok = torch.randint(0, V, (B, T + 1), generator=g)
        X, Y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
        _, loss = model(X, Y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    t_train = time.perf_counter() - t0
    model.eval()
    t1 = time.perf_counter()
    out = model.generate(torch.zeros(1, 1, dtype=torch.long), NEW_TOKENS)
    t_gen = time.perf_counter() - t1
    print(json.dumps({
        "impl": a.impl, "config": "char-gpt 6L/6H/384 ctx 256 vocab 65 dropout 0.2 batch 64, fp32, CPU",
        "params": n_params, "steps": a.steps, "train_seconds": round(t_train, 2),
        "tokens_per_second": round(a.steps * B * T / t_train, 1),
        "first_loss": round(losses[0], 4), "last_loss": round(losses[-1], 4),
        "generate_tokens": int(out.shape[1] - 1), "generate_seconds": round(t_gen, 2),
        "torch_threads": torch.get_num_threads(), "data": "synthetic (seeded uniform tokens)"}))


if __name__ == "__main__":
    main()
