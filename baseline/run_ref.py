"""Reference arm of the benchmark: the reference's unmodified `GPT` model driven exactly as its
DDP trainer drives it (nn/gpt2/train_ddp.py:71-103,134-143): seed 42, TF32 "high",
`torch.compile`, `DistributedDataParallel`, AdamW with the dim>=2 weight-decay rule and
`fused=True`, bf16 autocast, `clip_grad_norm_(1.0)`, cosine schedule.

The trainer script itself cannot be launched offline (it imports a streaming dataset and a
tokenizer that download at import time, nn/gpt2/data.py:5, nn/gpt2/hellaswag.py:8) and hard-codes
its hyper-parameters, so this driver imports `modules.py` from the installed copy of the
reference unchanged and supplies the benchmark's hyper-parameters (vocab 50304, lr 6e-4,
dropout 0, micro-batch 16x1024 accumulated to 524,288 tokens with `no_sync`).
None of this repository's kernels, models or engine are on this path.
"""
from __future__ import annotations

import contextlib
import importlib.util
import math
from pathlib import Path

import torch


def load_reference_modules(ref_dir: Path):
    spec = importlib.util.spec_from_file_location("z2h_reference_gpt2_modules", ref_dir / "modules.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def build_reference_step(ref_dir, model_kw, micro_b, seq, total_tokens, rank, world, local,
                         compile_model: bool = True):
    ref = load_reference_modules(Path(ref_dir))
    device = torch.device("cuda", local)
    torch.manual_seed(42)
    torch.set_float32_matmul_precision("high")
    config = ref.Config(vocab_size=model_kw["vocab_size"], block_size=model_kw["block_size"],
                        emb_dim=model_kw["emb_dim"], num_heads=model_kw["num_heads"],
                        num_layers=model_kw["num_layers"], dropout=0.0)
    model = ref.GPT(config).to(device)
    raw_model = model
    if compile_model:
        model = torch.compile(model)
    if world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP
        model = DDP(model, device_ids=[local])
    decay_params = [p for p in raw_model.parameters() if p.dim() >= 2]
    no_decay_params = [p for p in raw_model.parameters() if p.dim() < 2]
    lr_max, lr_min, warmup, steps_total = 6e-4, 6e-5, 128, 10_000
    optimizer = torch.optim.AdamW(
        [{"params": decay_params, "weight_decay": 0.1},
         {"params": no_decay_params, "weight_decay": 0.0}],
        lr=lr_max, betas=(0.9, 0.95), eps=1e-8, fused=True)

    def get_lr(step):
        if step < warmup:
            return lr_max * (step + 1) / warmup
        progress = (step - warmup) / (steps_total - warmup)
        return lr_min + (lr_max - lr_min) * 0.5 * (1 + math.cos(math.pi * progress))

    model.train()
    micro = total_tokens // (micro_b * seq * world)
    state = {"step": 0}

    def step(batches, read_loss: bool):
        for g in optimizer.param_groups:
            g["lr"] = get_lr(state["step"])
        optimizer.zero_grad(set_to_none=True)
        total = None
        n = len(batches)
        for i, (X, Y) in enumerate(batches):
            X = X.to(device, non_blocking=True)
            Y = Y.to(device, non_blocking=True)
            sync_ctx = model.no_sync() if (world > 1 and i < n - 1) else contextlib.nullcontext()
            with sync_ctx:
                with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
                    _, loss = model(X, Y)
                (loss / n).backward()
            total = loss.detach() / n if total is None else total + loss.detach() / n
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        optimizer.step()
        state["step"] += 1
        return float(total.item()) if read_loss else None

    return step, micro, (lambda: 0), "reference modules.GPT + torch.compile + DDP + fused AdamW"
