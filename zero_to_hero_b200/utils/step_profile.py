"""Runs a few micro-steps of the fused GPT-2 engine without CUDA graphs, so that a profiler
sees every kernel launch individually.

    python -m zero_to_hero_b200.utils.step_profile --preset gpt2-124m --micro-steps 2

Under Nsight Compute, capture the second micro-step (the first one also pays lazy module
loading): `ncu --metrics gpu__time_duration.sum --clock-control none -s <launches per
micro-step + 2> -c <launches per micro-step> --csv ...`. The script prints the launch count.
"""
from __future__ import annotations

import argparse

import torch

from ..config import apply_overrides, get_preset
from ..engine import GPT2TrainEngine
from ..ops import _lib


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="gpt2-124m")
    ap.add_argument("--micro-steps", type=int, default=2)
    ap.add_argument("--set", nargs="*", default=[], help="config overrides section.key=value")
    a = ap.parse_args()
    cfg = apply_overrides(get_preset(a.preset), a.set)
    cfg.train.use_cuda_graph = False
    eng = GPT2TrainEngine(cfg, "cuda")
    B, T, V = cfg.train.micro_batch, cfg.model.block_size, cfg.model.vocab_size
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, V, (B * T + 1,), generator=g)
    X, Y = tok[:-1].view(B, T).cuda(), tok[1:].view(B, T).cuda()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(a.micro_steps + 1)]
    ev[0].record()
    for i in range(a.micro_steps):
        eng.micro_step(X, Y, a.micro_steps)
        ev[i + 1].record()
    eng.optimizer_step()
    torch.cuda.synchronize()
    _lib.check_status()
    print(f"launches per micro-step: {eng.launches_per_micro_step}")
    for i in range(a.micro_steps):
        print(f"micro-step {i}: {ev[i].elapsed_time(ev[i + 1]):.3f} ms")
    print(f"loss {eng.read_loss():.4f}")


if __name__ == "__main__":
    main()
