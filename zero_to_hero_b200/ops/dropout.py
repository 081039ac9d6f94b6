"""Host restatement of the counter-based dropout masks of the CUDA kernels (csrc/common/dropout.cuh).

A mask is a pure function of (seed, site, element index): one 32-bit word per 4 consecutive
elements, one byte per element, kept when the byte is >= round(p * 256). These functions return the
same masks as torch tensors, so tests can run a plain PyTorch model with exactly the mask a kernel
used, and users can reproduce a training run's masks offline.
"""
from __future__ import annotations

import torch

_M32 = 0xFFFFFFFF
_M64 = 0xFFFFFFFFFFFFFFFF


def _site_seed(seed: int, site: int) -> tuple[int, int]:
    s = (seed + site * 0x9E3779B97F4A7C15) & _M64
    s ^= s >> 31
    s = (s * 0xBF58476D1CE4E5B9) & _M64
    s ^= s >> 29
    return s & _M32, (s >> 32) & _M32


def threshold_and_scale(p: float) -> tuple[int, float]:
    t = min(255, max(0, int(p * 256.0 + 0.5)))
    return t, 256.0 / (256.0 - t)


def _words(seed_lo: int, seed_hi: int, idx: torch.Tensor) -> torch.Tensor:
    """dropout_word() for a tensor of 64-bit word indices (int64, non-negative)."""
    lo = idx & _M32
    hi = (idx >> 32) & _M32
    x = (lo * 0x9E3779B1 + seed_lo) & _M32
    y = (hi * 0x85EBCA77 + seed_hi) & _M32
    x = x ^ y
    x = x ^ (x >> 16)
    x = (x * 0x85EBCA6B) & _M32
    x = x ^ (x >> 13)
    x = (x * 0xC2B2AE35) & _M32
    x = x ^ (x >> 16)
    x = (x + ((y * 0x27D4EB2F) & _M32)) & _M32
    x = x ^ (x >> 15)
    x = (x * 0x2C1B3C6D) & _M32
    x = x ^ (x >> 12)
    return x


def elementwise_keep(n: int, p: float, seed: int, site: int, device="cpu") -> torch.Tensor:
    """Keep mask (bool [n]) of `dropout_apply` over n contiguous elements."""
    lo, hi = _site_seed(seed, site)
    t, _ = threshold_and_scale(p)
    e = torch.arange(n, dtype=torch.int64, device=device)
    w = _words(lo, hi, e >> 2)
    return ((w >> (8 * (e & 3))) & 0xFF) >= t


def attention_keep(B: int, H: int, T: int, p: float, seed: int, site: int, device="cpu") -> torch.Tensor:
    """Keep mask (bool [B, H, T, T], query x key) of the attention kernels' probability dropout."""
    lo, hi = _site_seed(seed, site)
    t, _ = threshold_and_scale(p)
    wpr = (T + 3) // 4
    bh = torch.arange(B * H, dtype=torch.int64, device=device).view(B * H, 1, 1)
    q = torch.arange(T, dtype=torch.int64, device=device).view(1, T, 1)
    k = torch.arange(T, dtype=torch.int64, device=device).view(1, 1, T)
    w = _words(lo, hi, (bh * T + q) * wpr + (k >> 2))
    return (((w >> (8 * (k & 3))) & 0xFF) >= t).view(B, H, T, T)
