"""AdamW parameter groups and a module-level optimizer wrapper.

`param_groups` reproduces the reference's grouping (nn/gpt2/train.py:73-84): tensors with
`dim() >= 2` get weight decay, everything else (biases, LayerNorm weights) does not.
`build_optimizer` returns a torch AdamW over those groups for the PyTorch path (fused on CUDA,
as in the reference); the fused engine applies the same rule through its own kernel
(csrc/optim/adamw.cu) over flat buffers.
"""
from __future__ import annotations

import torch


def param_groups(model: torch.nn.Module, weight_decay: float) -> list[dict]:
    seen: set[int] = set()
    decay, no_decay = [], []
    for p in model.parameters():
        if id(p) in seen or not p.requires_grad:
            continue
        seen.add(id(p))
        (decay if p.dim() >= 2 else no_decay).append(p)
    return [
        {"params": decay, "weight_decay": weight_decay},
        {"params": no_decay, "weight_decay": 0.0},
    ]


def build_optimizer(model: torch.nn.Module, optim_cfg, device_type: str | None = None):
    groups = param_groups(model, optim_cfg.weight_decay)
    if device_type is None:
        device_type = next(model.parameters()).device.type
    kwargs = {"fused": True} if device_type == "cuda" else {}
    return torch.optim.AdamW(groups, lr=optim_cfg.lr_max, betas=(optim_cfg.beta1, optim_cfg.beta2),
                             eps=optim_cfg.eps, **kwargs)


def set_lr(optimizer: torch.optim.Optimizer, lr: float) -> None:
    for g in optimizer.param_groups:
        g["lr"] = lr
