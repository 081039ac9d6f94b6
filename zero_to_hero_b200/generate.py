"""Sampling entry point: load a checkpoint (or random weights) and generate tokens.

    python -m zero_to_hero_b200.generate --preset gpt2-tiny --tokens 64 --top-k 50
    python -m zero_to_hero_b200.generate --checkpoint run/step00001000.pt --prompt-ids 1,2,3

Mirrors `GPT.generate` of the reference (nn/gpt2/modules.py:121-137) and the char-level
script's final sampling (nn/gpt/3_gpt.py:245-248).
"""
from __future__ import annotations

import argparse

import torch

from .config import Config, apply_overrides, get_preset
from .train import build_module


def sample(cfg: Config, state_dict=None, prompt=None, tokens: int = 64, temperature: float = 1.0,
           top_k: int | None = None, seed: int = 0, device: str | None = None) -> torch.Tensor:
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    model = build_module(cfg).to(device).eval()
    if state_dict is not None:
        model.load_state_dict(state_dict, strict=False)
    X = torch.zeros(1, 1, dtype=torch.long) if prompt is None else torch.tensor([prompt], dtype=torch.long)
    if cfg.model.kind == "char":
        gen = torch.Generator(device=device).manual_seed(seed)
        return model.generate(X.to(device), tokens, generator=gen)
    if torch.device(device).type == "cuda":
        # no generator object: on a GPU `sample_next` then runs the fused temperature / top-k /
        # multinomial kernel (csrc/sample/sample_topk.cu), seeded from torch's global generator
        torch.manual_seed(seed)
        return model.generate(X.to(device), tokens, temperature=temperature, top_k=top_k)
    gen = torch.Generator(device=device).manual_seed(seed)
    return model.generate(X.to(device), tokens, temperature=temperature, top_k=top_k, generator=gen)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="gpt2-tiny")
    ap.add_argument("--checkpoint", default="")
    ap.add_argument("--prompt-ids", default="")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    sd = None
    if a.checkpoint:
        from .utils.checkpoint import load_checkpoint
        ck = load_checkpoint(a.checkpoint)
        cfg = Config.from_dict(ck["config"]) if ck.get("config") else get_preset(a.preset)
        sd = ck["model"]
    else:
        cfg = get_preset(a.preset)
    cfg = apply_overrides(cfg, a.overrides)
    prompt = [int(t) for t in a.prompt_ids.split(",")] if a.prompt_ids else None
    out = sample(cfg, sd, prompt, a.tokens, a.temperature, a.top_k, a.seed)
    print(out[0].tolist())


if __name__ == "__main__":
    main()
