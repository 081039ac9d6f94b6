"""Seeded synthetic token streams.

The reference streams FineWeb-Edu through tiktoken (nn/gpt2/data.py:11-49), which needs the
network; benchmarks and tests here use uniform random tokens of the same shape instead:
`next_batch()` returns X, Y of shape [B, T] with Y = X shifted by one, exactly as the
reference loader builds them from B*T+1 consecutive tokens (nn/gpt2/data.py:42-49).
Batches are produced on the host in pinned memory so that the host->device copy is part of
what a training step pays for, as it is with the reference loader.
"""
from __future__ import annotations

import torch


class SyntheticLoader:
    def __init__(self, split: str, batch_size: int, block_size: int, vocab_size: int,
                 device: torch.device | str = "cpu", rank: int = 0, world_size: int = 1,
                 seed: int = 1234, pin: bool | None = None):
        self.batch_size, self.block_size, self.vocab_size = batch_size, block_size, vocab_size
        self.device = torch.device(device)
        salt = {"train": 0, "val": 1}.get(split, 2)
        # validation is not sharded (nn/gpt2/train_ddp.py:77); training is, by rank
        r = rank if split == "train" else 0
        self._rank = r
        self.gen = torch.Generator(device="cpu").manual_seed(seed + 1000003 * salt + 7919 * r)
        self.pin = (self.device.type == "cuda") if pin is None else pin
        self.cursor = 0

    def next_host_batch(self) -> tuple[torch.Tensor, torch.Tensor]:
        n = self.batch_size * self.block_size + 1
        tokens = torch.randint(0, self.vocab_size, (n,), generator=self.gen, dtype=torch.int64)
        self.cursor += n - 1
        X = tokens[:-1].view(self.batch_size, self.block_size)
        Y = tokens[1:].view(self.batch_size, self.block_size)
        if self.pin:
            X, Y = X.contiguous().pin_memory(), Y.contiguous().pin_memory()
        return X, Y

    def next_batch(self) -> tuple[torch.Tensor, torch.Tensor]:
        X, Y = self.next_host_batch()
        if self.device.type == "cpu":
            return X, Y
        return X.to(self.device, non_blocking=True), Y.to(self.device, non_blocking=True)

    def state(self) -> dict:
        return {"cursor": self.cursor, "rng": self.gen.get_state()}

    def load_state(self, st: dict) -> None:
        if st.get("reshard"):
            # another job size: a rank that existed before carries on with that rank's generator, a
            # new rank keeps the fresh stream of its own index; all take the furthest cursor
            states = st["per_rank"]
            self.cursor = max(int(s["cursor"]) for s in states)
            if self._rank < len(states):
                self.gen.set_state(states[self._rank]["rng"])
            return
        self.cursor = st["cursor"]
        self.gen.set_state(st["rng"])
