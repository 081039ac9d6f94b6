"""Loaders that read from local files (no network).

`CharTextLoader` reproduces the batching of the reference's char-level scripts
(nn/gpt/3_gpt.py:184-202): a 90/10 train/val split of one text file and random-offset
windows of `block_size` characters with targets shifted by one.
`TokenFileLoader` streams a flat token file (uint16/int32 `.bin` or a torch `.pt` tensor)
sharded by rank with wrap-around, the offline stand-in for the reference's FineWeb-Edu stream
(nn/gpt2/data.py:11-49).
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from ..models.gpt import Vocab


class CharTextLoader:
    def __init__(self, path: str | Path, batch_size: int, block_size: int,
                 device: torch.device | str = "cpu", seed: int = 42, train_frac: float = 0.9):
        text = Path(path).read_text(encoding="utf-8")
        self.vocab = Vocab(text)
        data = torch.tensor(self.vocab.encode(text), dtype=torch.long)
        n = int(train_frac * len(data))
        self.splits = {"train": data[:n], "val": data[n:]}
        self.batch_size, self.block_size = batch_size, block_size
        self.device = torch.device(device)
        self.gen = torch.Generator().manual_seed(seed)

    def get_batch(self, split: str = "train"):
        data = self.splits[split]
        ix = torch.randint(len(data) - self.block_size, (self.batch_size,), generator=self.gen)
        offsets = torch.arange(self.block_size)
        X = data[ix.unsqueeze(1) + offsets]
        Y = data[ix.unsqueeze(1) + offsets + 1]
        return X.to(self.device), Y.to(self.device)

    next_batch = get_batch


class TokenFileLoader:
    def __init__(self, path: str | Path, batch_size: int, block_size: int, rank: int = 0,
                 world_size: int = 1, dtype: str = "uint16", pin: bool = False,
                 split: str = "all", val_frac: float = 0.0):
        """`split="train"` reads the head of the file and `split="val"` its last `val_frac`
        (the reference holds out its first 16,384 documents, nn/gpt2/data.py:23-24); "all" reads
        everything."""
        path = Path(path)
        if path.suffix == ".pt":
            tokens = torch.load(path).to(torch.int64)
        else:
            tokens = torch.from_numpy(np.fromfile(path, dtype=np.dtype(dtype)).astype(np.int64))
        if split != "all" and val_frac > 0.0:
            n_val = max(batch_size * block_size + 1, int(len(tokens) * val_frac))
            n_val = min(n_val, len(tokens) // 2)
            tokens = tokens[-n_val:] if split == "val" else tokens[:-n_val]
        self.tokens = tokens
        self.batch_size, self.block_size = batch_size, block_size
        self.rank, self.world_size = rank, world_size
        self.pin = pin
        self.span = batch_size * block_size
        if len(self.tokens) < self.span * world_size + 1:
            raise ValueError("token file is shorter than one global batch")
        self.cursor = rank * self.span

    def next_host_batch(self):
        n = self.span
        if self.cursor + n + 1 > len(self.tokens):
            self.cursor = self.rank * n  # wrap around, as the reference restarts its iterator
        tok = self.tokens[self.cursor:self.cursor + n + 1]
        self.cursor += n * self.world_size
        X = tok[:-1].view(self.batch_size, self.block_size).contiguous()
        Y = tok[1:].view(self.batch_size, self.block_size).contiguous()
        if self.pin:
            X, Y = X.pin_memory(), Y.pin_memory()
        return X, Y

    next_batch = next_host_batch

    def state(self):
        return {"cursor": self.cursor}

    def load_state(self, st):
        if st.get("reshard"):
            # Saved by a job of another size. Rank r of W ranks sits at r*span + k*span*W after k
            # batches, so the smallest saved cursor, rounded down to a whole global batch of the old
            # job, is where the stream as a whole stands; this rank takes its own stride from there.
            old_world = int(st["old_world"])
            lowest = min(int(s["cursor"]) for s in st["per_rank"])
            consumed = lowest - lowest % (self.span * old_world)
            self.cursor = consumed + self.rank * self.span
            return
        self.cursor = st["cursor"]
