"""Config presets/overrides, LR schedule and AdamW grouping (CPU)."""
import math

import pytest
import torch

from zero_to_hero_b200.config import Config, apply_overrides, get_preset, nice
from zero_to_hero_b200.models.gpt2 import GPT2
from zero_to_hero_b200.optim.adamw import build_optimizer, param_groups
from zero_to_hero_b200.optim.schedule import get_lr


def test_nice_matches_reference_padding():
    assert nice(50257, 256) == 50432  # nn/gpt2/train_ddp.py:24-28
    assert nice(50257, 128) == 50304


def test_presets_and_overrides():
    cfg = get_preset("gpt2-124m")
    assert (cfg.model.num_layers, cfg.model.num_heads, cfg.model.emb_dim) == (12, 12, 768)
    assert cfg.model.vocab_size == 50304 and cfg.train.total_batch_tokens == 524288
    cfg = apply_overrides(cfg, ["model.num_layers=4", "optim.lr_max=3e-4", "train.use_cuda_graph=false"])
    assert cfg.model.num_layers == 4 and cfg.optim.lr_max == 3e-4 and cfg.train.use_cuda_graph is False
    with pytest.raises(KeyError):
        apply_overrides(cfg, ["model.nope=1"])
    assert Config.from_dict(cfg.to_dict()).model.num_layers == 4
    big = get_preset("gpt2-1.5b").model
    assert big.emb_dim // big.num_heads == 64 and big.num_layers == 48
    char = get_preset("char-gpt").model
    assert (char.num_layers, char.num_heads, char.emb_dim, char.block_size, char.vocab_size) == (6, 6, 384, 256, 65)


def test_lr_schedule_matches_reference_formula():
    lr_max, lr_min, warm, steps = 3e-4, 3e-5, 128, 1000

    def ref(step):  # nn/gpt2/train_ddp.py:124-129
        if step < warm:
            return lr_max * (step + 1) / warm
        progress = (step - warm) / (steps - warm)
        return lr_min + (lr_max - lr_min) * 0.5 * (1 + math.cos(math.pi * progress))

    for s in [0, 1, 127, 128, 500, 999]:
        assert get_lr(s, lr_max, lr_min, warm, steps) == pytest.approx(ref(s), rel=1e-12)


def test_param_groups_dim_rule():
    cfg = get_preset("gpt2-tiny")
    model = GPT2(cfg.model)
    groups = param_groups(model, 0.1)
    assert all(p.dim() >= 2 for p in groups[0]["params"]) and groups[0]["weight_decay"] == 0.1
    assert all(p.dim() < 2 for p in groups[1]["params"]) and groups[1]["weight_decay"] == 0.0
    n = sum(p.numel() for g in groups for p in g["params"])
    assert n == sum(p.numel() for p in model.parameters())  # tied weight counted once
    opt = build_optimizer(model, cfg.optim)
    assert opt.param_groups[0]["betas"] == (0.9, 0.95)


def test_pick_split_k_fills_whole_waves():
    """Split-K factors for the weight-gradient shapes of GPT-2 124M at 16,384 tokens: the factor
    must keep the 74 CTA pairs busy for whole waves, and huge outputs need no split."""
    import math
    from zero_to_hero_b200.ops.functional import pick_split_k

    def tiles(n_out, k_in):
        return math.ceil(n_out / 128) * math.ceil(k_in / 256)

    kb = 16384 // 64
    for n_out, k_in in ((2304, 768), (768, 768), (3072, 768), (768, 3072)):
        s = pick_split_k(tiles(n_out, k_in), kb)
        pair_tiles = math.ceil(tiles(n_out, k_in) / 2)
        waves = pair_tiles * s / 74
        assert s >= 1 and kb // s >= 16
        assert math.ceil(waves) - waves < 0.15, (n_out, k_in, s, waves)
    assert pick_split_k(tiles(50304, 768), kb) == 1
    assert pick_split_k(4, 8) == 1  # K too short to split
