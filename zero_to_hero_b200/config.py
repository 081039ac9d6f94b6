"""Configuration dataclasses, named presets and `key=value` overrides.

The reference keeps its training configuration in module-level constants
(nn/gpt2/train.py:15-29, nn/gpt2/train_ddp.py:28-42, nn/gpt/3_gpt.py:153-162) and only the
model in a dataclass (nn/gpt2/modules.py:7-14). Here everything is a dataclass tree that can
be built from a preset name and overridden from the command line.
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field, fields, is_dataclass
from typing import Any


def nice(n: int, multiple: int) -> int:
    """Round `n` up to a multiple (the reference's vocab padding, nn/gpt2/train_ddp.py:24-28)."""
    return ((n + multiple - 1) // multiple) * multiple


@dataclass
class ModelConfig:
    vocab_size: int = 50257
    block_size: int = 1024
    emb_dim: int = 768
    num_heads: int = 12
    num_layers: int = 12
    dropout: float = 0.0
    ln_bias: bool = False       # the reference's GPT-2 LayerNorms carry no bias
    kind: str = "gpt2"          # "gpt2" | "char" (per-head attention, ReLU MLP, untied head)

    @property
    def head_dim(self) -> int:
        return self.emb_dim // self.num_heads

    @property
    def padded_vocab(self) -> int:
        """Row count of the logits buffer: vocabulary rounded up to 8 columns (16 bytes)."""
        return nice(self.vocab_size, 8)


@dataclass
class OptimConfig:
    lr_max: float = 6e-4
    lr_min_ratio: float = 0.1
    warmup_steps: int = 128
    total_steps: int = 10_000
    schedule: str = "cosine"    # "cosine" | "constant"
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    clip_norm: float = 1.0      # <= 0 disables clipping


@dataclass
class TrainConfig:
    micro_batch: int = 16
    total_batch_tokens: int = 524_288
    steps: int = 20
    seed: int = 42
    dtype: str = "bf16"         # compute dtype of the fused engine; "fp32" = PyTorch path
    eval_interval: int = 256
    eval_batches: int = 1
    log_interval: int = 1
    data: str = "synthetic"     # "synthetic" | "char:<path>" | "tokens:<path>"
    val_frac: float = 0.05      # tokens:<path> only: tail of the file held out for validation
    hellaswag: str = ""         # JSONL of pre-tokenised HellaSwag examples; scored at eval time
    checkpoint_dir: str = ""
    checkpoint_interval: int = 0
    # resume a checkpoint written by a job with another number of ranks: parameters and moments load
    # into any world size, the data cursors are re-sharded (engine.select_rank_state)
    elastic_resume: bool = False
    use_cuda_graph: bool = True
    overlap_wgrad: bool = True  # weight-gradient GEMMs on a second stream (fills the tails of the data-gradient chain)
    # Bitwise reproducible steps: every accumulation that normally meets in atomics runs in a fixed
    # order instead (split-K weight gradients folded slice by slice, attention dQ one KV tile per launch,
    # bias and embedding gradients by ordered sums). 0.86x the speed on the 124M model.
    deterministic: bool = False
    log_jsonl: str = ""


@dataclass
class DistConfig:
    backend: str = "auto"       # "nccl" on GPU, "gloo" on CPU
    fused_allreduce: bool = True  # own P2P reduce-scatter + AdamW + all-gather kernel
    nvls: bool = False          # multimem flavour of the fused kernel
    bucket_mb: float = 32.0     # gradient buckets reduced while backward still runs; 0 = one reduce after it
    timeout_s: float = 600.0    # process-group timeout and heartbeat patience (host side)
    device_wait_s: float = 2.0  # budget of a kernel's wait for a peer's signal (device side)
    heartbeat_interval: int = 1  # steps between host heartbeat checks; 0 = off


@dataclass
class Config:
    model: ModelConfig = field(default_factory=ModelConfig)
    optim: OptimConfig = field(default_factory=OptimConfig)
    train: TrainConfig = field(default_factory=TrainConfig)
    dist: DistConfig = field(default_factory=DistConfig)

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), indent=2)

    @staticmethod
    def from_dict(d: dict) -> "Config":
        cfg = Config()
        for section, values in d.items():
            sub = getattr(cfg, section)
            for k, v in values.items():
                setattr(sub, k, v)
        return cfg


def _gpt2(vocab, layers, heads, dim) -> ModelConfig:
    return ModelConfig(vocab_size=vocab, block_size=1024, emb_dim=dim, num_heads=heads,
                       num_layers=layers, dropout=0.0)


PRESETS: dict[str, Any] = {
    # char-level GPT on CPU: 6 layers, 6 heads, 384 wide, context 256, vocab 65, batch 64
    "char-gpt": lambda: Config(
        model=ModelConfig(vocab_size=65, block_size=256, emb_dim=384, num_heads=6, num_layers=6,
                          dropout=0.2, ln_bias=True, kind="char"),
        optim=OptimConfig(lr_max=3e-4, schedule="constant", warmup_steps=0, weight_decay=0.01,
                          clip_norm=0.0, beta2=0.999),
        train=TrainConfig(micro_batch=64, total_batch_tokens=64 * 256, steps=20, dtype="fp32")),
    "gpt2-124m": lambda: Config(
        model=_gpt2(50304, 12, 12, 768),
        train=TrainConfig(micro_batch=16, total_batch_tokens=524_288)),
    "gpt2-350m": lambda: Config(
        model=_gpt2(50304, 24, 16, 1024),
        train=TrainConfig(micro_batch=8, total_batch_tokens=524_288)),
    "gpt2-1.5b": lambda: Config(
        model=_gpt2(50304, 48, 25, 1600),
        train=TrainConfig(micro_batch=8, total_batch_tokens=1_048_576)),
    # tiny model for tests and smoke runs
    "gpt2-tiny": lambda: Config(
        model=ModelConfig(vocab_size=512, block_size=128, emb_dim=128, num_heads=2, num_layers=2),
        optim=OptimConfig(warmup_steps=2, total_steps=100),
        train=TrainConfig(micro_batch=4, total_batch_tokens=4 * 128 * 2, steps=4)),
}


def get_preset(name: str) -> Config:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; available: {sorted(PRESETS)}")
    return PRESETS[name]()


def _coerce(old: Any, text: str) -> Any:
    if isinstance(old, bool):
        return text.lower() in ("1", "true", "yes", "on")
    if isinstance(old, int):
        return int(float(text)) if ("e" in text.lower() or "." in text) else int(text.replace("_", ""))
    if isinstance(old, float):
        return float(text)
    return text


def apply_overrides(cfg: Config, overrides: list[str]) -> Config:
    """Apply `section.key=value` strings, e.g. `model.num_layers=4 optim.lr_max=3e-4`."""
    for item in overrides:
        if "=" not in item:
            raise ValueError(f"override {item!r} is not of the form section.key=value")
        key, text = item.split("=", 1)
        parts = key.split(".")
        if len(parts) != 2:
            raise ValueError(f"override key {key!r} must be section.key")
        sub = getattr(cfg, parts[0], None)
        if sub is None or not is_dataclass(sub) or parts[1] not in {f.name for f in fields(sub)}:
            raise KeyError(f"unknown config key {key!r}")
        setattr(sub, parts[1], _coerce(getattr(sub, parts[1]), text))
    return cfg
