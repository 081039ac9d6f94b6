"""Step logging: one human-readable line (the reference's format, nn/gpt2/train_ddp.py:160-175)
and an optional JSONL record per step; only rank 0 writes."""
from __future__ import annotations

import json
import time
from pathlib import Path


class StepLogger:
    def __init__(self, jsonl_path: str = "", is_master: bool = True):
        self.is_master = is_master
        self.f = open(Path(jsonl_path), "a") if (jsonl_path and is_master) else None

    def log(self, step: int, **fields) -> str:
        parts = [f"step {step:8d}"]
        for k, v in fields.items():
            if isinstance(v, float):
                if k == "lr":
                    parts.append(f"{k} {v:.2e}")
                elif k.endswith("tok_s"):
                    parts.append(f"{v:8.0f} tok/s")
                elif k.endswith("ms"):
                    parts.append(f"{v:8.2f}ms")
                else:
                    parts.append(f"{k} {v:8.4f}")
            else:
                parts.append(f"{k} {v}")
        line = " | ".join(parts)
        if self.is_master:
            print(line, flush=True)
            if self.f:
                self.f.write(json.dumps({"step": step, "time": time.time(), **fields}) + "\n")
                self.f.flush()
        return line

    def close(self):
        if self.f:
            self.f.close()
