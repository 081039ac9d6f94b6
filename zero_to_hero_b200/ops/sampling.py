"""Next-token sampling: temperature, top-k, softmax, multinomial
(nn/gpt2/modules.py:130-135; the char-level models sample without temperature/top-k,
nn/gpt/3_gpt.py:141-149)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


_counter = 0


def sample_topk_native(logits: torch.Tensor, temperature: float = 1.0, top_k: int | None = None,
                       seed: int = 0, offset: int = 0) -> torch.Tensor:
    """One fused kernel per batch (csrc/sample/sample_topk.cu): fp32 CUDA logits [B, V] -> ids [B, 1].
    Deterministic in (logits, temperature, top_k, seed, offset)."""
    import ctypes
    from . import _lib
    lib = _lib.cuda_lib()
    fn = lib.z2h_sample_topk
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_longlong,
                   ctypes.c_float, ctypes.c_int, ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_void_p]
    x = logits.float().contiguous()
    B, V = x.shape
    out = torch.zeros(B, dtype=torch.int64, device=x.device)
    rc = fn(_lib.ptr(x), _lib.ptr(out), B, V, x.stride(0), float(temperature), int(top_k or 0),
            int(seed) & (2**64 - 1), int(offset), _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"z2h_sample_topk failed with code {rc}")
    return out.unsqueeze(1)


def sample_next(logits: torch.Tensor, temperature: float = 1.0, top_k: int | None = None,
                generator: torch.Generator | None = None) -> torch.Tensor:
    """logits [B, V] -> sampled ids [B, 1]. On a GPU without an explicit generator the fused
    kernel is used, seeded from torch's global CPU generator so `torch.manual_seed` reproduces."""
    global _counter
    if logits.is_cuda and generator is None:
        seed = int(torch.randint(0, 2**62, (1,)).item())
        _counter += logits.shape[0]
        return sample_topk_native(logits, temperature, top_k, seed, _counter)
    logits = logits / temperature
    if top_k is not None:
        v, _ = torch.topk(logits, min(top_k, logits.size(-1)))
        logits = logits.masked_fill(logits < v[:, [-1]], -float("inf"))
    probs = F.softmax(logits, dim=-1)
    return torch.multinomial(probs, num_samples=1, generator=generator)
