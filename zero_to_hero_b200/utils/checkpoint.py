"""Checkpoints in the GPT-2 state_dict layout.

The reference never saves anything (no torch.save/load in nn/gpt2). Here a checkpoint is one
`torch.save` file holding

  model      fp32 tensors under Hugging Face GPT-2 names, Linear weights as (out, in)
  optim      AdamW state: step count, first/second moments as flat vectors (engine layout) or
             the torch optimizer's state_dict (module path)
  step, rng  optimizer step, CPU/CUDA RNG states
  data       loader cursor / generator state
  config     the Config tree as a dict

plus converters between three naming schemes of the same network:
  * this package / Hugging Face (`transformer.h.0.attn.c_attn.weight`, ...),
  * the reference's module names (`blocks.0.attn.proj_heads.weight`, ...,
    nn/gpt2/modules.py:21-22,48-52,62-65,77-82),
  * Hugging Face's on-disk GPT-2 format, whose Conv1D weights are stored (in, out) and whose
    LayerNorms carry biases (exported as zeros; on import they must be zero unless the model
    was built with `ln_bias=True`).
"""
from __future__ import annotations

import os
import re
from pathlib import Path
from typing import Any

import torch

_BLOCK_MAP = {
    "ln1.weight": "ln_1.weight", "ln1.bias": "ln_1.bias",
    "attn.proj_heads.weight": "attn.c_attn.weight", "attn.proj_heads.bias": "attn.c_attn.bias",
    "attn.proj_output.weight": "attn.c_proj.weight", "attn.proj_output.bias": "attn.c_proj.bias",
    "ln2.weight": "ln_2.weight", "ln2.bias": "ln_2.bias",
    "ff.ff.0.weight": "mlp.c_fc.weight", "ff.ff.0.bias": "mlp.c_fc.bias",
    "ff.ff.2.weight": "mlp.c_proj.weight", "ff.ff.2.bias": "mlp.c_proj.bias",
}
_TOP_MAP = {
    "tok_to_emb.weight": "transformer.wte.weight", "pos_to_emb.weight": "transformer.wpe.weight",
    "ln.weight": "transformer.ln_f.weight", "ln.bias": "transformer.ln_f.bias",
    "head.weight": "lm_head.weight",
}
_CONV1D = ("attn.c_attn.weight", "attn.c_proj.weight", "mlp.c_fc.weight", "mlp.c_proj.weight")


def _strip_prefixes(key: str) -> str:
    for p in ("module.", "_orig_mod."):
        while key.startswith(p):
            key = key[len(p):]
    return key


def reference_to_hf_name(key: str) -> str:
    key = _strip_prefixes(key)
    if key in _TOP_MAP:
        return _TOP_MAP[key]
    m = re.match(r"blocks\.(\d+)\.(.+)$", key)
    if m and m.group(2) in _BLOCK_MAP:
        return f"transformer.h.{m.group(1)}.{_BLOCK_MAP[m.group(2)]}"
    raise KeyError(f"not a reference GPT parameter name: {key}")


def hf_to_reference_name(key: str) -> str:
    inv_top = {v: k for k, v in _TOP_MAP.items()}
    inv_block = {v: k for k, v in _BLOCK_MAP.items()}
    if key in inv_top:
        return inv_top[key]
    m = re.match(r"transformer\.h\.(\d+)\.(.+)$", key)
    if m and m.group(2) in inv_block:
        return f"blocks.{m.group(1)}.{inv_block[m.group(2)]}"
    raise KeyError(f"not a GPT-2 parameter name: {key}")


def from_reference_state_dict(sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Reference `GPT.state_dict()` -> this package's names (tensors shared, not copied)."""
    return {reference_to_hf_name(k): v for k, v in sd.items()}


def to_reference_state_dict(sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    return {hf_to_reference_name(k): v for k, v in sd.items()}


def to_hf_disk_format(sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """(out, in) Linear weights -> Conv1D (in, out); add zero LayerNorm biases if absent."""
    out = {}
    for k, v in sd.items():
        out[k] = v.t().contiguous() if k.endswith(_CONV1D) else v
    for k in list(out):
        if k.endswith(("ln_1.weight", "ln_2.weight", "ln_f.weight")):
            b = k[:-len("weight")] + "bias"
            if b not in out:
                out[b] = torch.zeros_like(out[k])
    return out


def from_hf_disk_format(sd: dict[str, torch.Tensor], ln_bias: bool = False) -> dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        if k.endswith(".attn.bias") or k.endswith(".attn.masked_bias"):
            continue  # causal-mask buffers of the HF implementation
        if k.endswith(("ln_1.bias", "ln_2.bias", "ln_f.bias")) and not ln_bias:
            if v.abs().max().item() != 0.0:
                raise ValueError(f"{k} is non-zero but the model has no LayerNorm bias "
                                 "(build it with ln_bias=True)")
            continue
        out[k] = v.t().contiguous() if k.endswith(_CONV1D) else v
    if "lm_head.weight" not in out and "transformer.wte.weight" in out:
        out["lm_head.weight"] = out["transformer.wte.weight"]
    return out


def rng_state() -> dict[str, Any]:
    st = {"cpu": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state_all()
    return st


def set_rng_state(st: dict[str, Any]) -> None:
    torch.set_rng_state(st["cpu"])
    if "cuda" in st and torch.cuda.is_available():
        try:
            torch.cuda.set_rng_state_all(st["cuda"])
        except RuntimeError:
            pass  # different number of devices than at save time


def save_checkpoint(path: str | os.PathLike, model_sd: dict[str, torch.Tensor], optim: Any,
                    step: int, data_state: dict | None = None, config: dict | None = None,
                    extra: dict | None = None) -> None:
    """Atomic write (tmp file + rename) of one checkpoint."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    payload = {
        "format": "z2h-gpt2-v1",
        "model": {k: v.detach().to("cpu", torch.float32) for k, v in model_sd.items()},
        "optim": optim, "step": step, "rng": rng_state(), "data": data_state, "config": config,
        "extra": extra or {},
    }
    tmp = path.with_suffix(path.suffix + ".tmp")
    torch.save(payload, tmp)
    os.replace(tmp, path)


def load_checkpoint(path: str | os.PathLike, map_location="cpu") -> dict:
    ck = torch.load(Path(path), map_location=map_location, weights_only=False)
    if ck.get("format") != "z2h-gpt2-v1":
        raise ValueError(f"{path} is not a z2h checkpoint")
    return ck
