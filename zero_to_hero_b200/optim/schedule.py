"""Learning-rate schedule: linear warm-up then cosine decay to `lr_min`.

Same form as `get_lr` of the reference trainers (nn/gpt2/train.py:106-111,
nn/gpt2/train_ddp.py:124-129): lr_max * (step + 1) / warmup during warm-up, afterwards
lr_min + (lr_max - lr_min) * 0.5 * (1 + cos(pi * progress)).
"""
from __future__ import annotations

import math


def get_lr(step: int, lr_max: float, lr_min: float, warmup_steps: int, total_steps: int,
           schedule: str = "cosine") -> float:
    if schedule == "constant":
        return lr_max
    if step < warmup_steps:
        return lr_max * (step + 1) / warmup_steps
    if total_steps <= warmup_steps:
        return lr_min
    progress = min(1.0, (step - warmup_steps) / (total_steps - warmup_steps))
    cosine = 0.5 * (1.0 + math.cos(math.pi * progress))
    return lr_min + (lr_max - lr_min) * cosine


def lr_for(step: int, optim_cfg) -> float:
    return get_lr(step, optim_cfg.lr_max, optim_cfg.lr_max * optim_cfg.lr_min_ratio,
                  optim_cfg.warmup_steps, optim_cfg.total_steps, optim_cfg.schedule)
