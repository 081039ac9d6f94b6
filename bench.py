"""Headline benchmark: GPT-2 124M training tokens/sec on N B200s of one node.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference model + torch DDP stack

One step = one optimizer step over 524,288 tokens: micro-batches of 16 x 1024 tokens per rank,
accumulated (32 / N micro-steps per rank), then grad-norm clip + AdamW. Tokens are seeded
uniform integers, weights are random-init, dropout is 0 on both arms.

Two timings are taken, each over exactly `--steps` steps after `--warmup` untimed ones, with a
barrier + device synchronize on both sides and the max over ranks:
  * `value`     device time (CUDA events) with the token batches already resident on the GPU;
  * `e2e.value` through the public API with every micro-batch copied from pinned host memory
                and the step's loss read back to the host every step.
Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MODEL = dict(vocab_size=50304, block_size=1024, emb_dim=768, num_heads=12, num_layers=12)
MICRO_B, SEQ, TOTAL_TOKENS = 16, 1024, 524_288


class ClockSampler:
    """Samples SM clocks / throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n_gpus:
        if world == 1 and n_gpus > 1:
            raise SystemExit(f"--gpus {n_gpus} needs a torchrun launch with {n_gpus} ranks")
        n_gpus = world
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync(world: int):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def make_host_batches(n: int, seed: int, vocab: int):
    """n pinned (X, Y) micro-batches of seeded uniform tokens, Y = X shifted by one."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        tok = torch.randint(0, vocab, (MICRO_B * SEQ + 1,), generator=g, dtype=torch.int64)
        out.append((tok[:-1].view(MICRO_B, SEQ).contiguous().pin_memory(),
                    tok[1:].view(MICRO_B, SEQ).contiguous().pin_memory()))
    return out


# ---------------------------------------------------------------------------------------------
# arm 1: this framework
# ---------------------------------------------------------------------------------------------
def build_ours(rank, world, local):
    from zero_to_hero_b200.config import get_preset
    from zero_to_hero_b200.engine import GPT2TrainEngine

    cfg = get_preset("gpt2-124m")
    for k, v in MODEL.items():
        setattr(cfg.model, k, v)
    cfg.train.micro_batch = MICRO_B
    cfg.train.total_batch_tokens = TOTAL_TOKENS
    if "Z2H_OVERLAP" in os.environ:  # A/B switch for the two-stream backward schedule
        cfg.train.overlap_wgrad = os.environ["Z2H_OVERLAP"] == "1"
    comm = None
    if world > 1:
        from zero_to_hero_b200.parallel.fused_ddp import FusedDDP
        # Z2H_NVLS=1 selects the multimem flavour of the fused reduce-scatter + AdamW + all-gather
        comm = FusedDDP(torch.device("cuda", local), nvls=os.environ.get("Z2H_NVLS", "0") == "1")
    eng = GPT2TrainEngine(cfg, device=torch.device("cuda", local), comm=comm)
    micro = TOTAL_TOKENS // (MICRO_B * SEQ * world)

    def step(batches, read_loss: bool):
        eng.train_step(batches)
        return eng.read_loss() if read_loss else None

    return step, micro, lambda: eng.kernel_launches_per_step(micro), "fused-engine"


# ---------------------------------------------------------------------------------------------
# arm 2: the unmodified reference model driven as its DDP trainer drives it
# ---------------------------------------------------------------------------------------------
def build_reference(rank, world, local):
    ref_dir = ROOT / "baseline" / "_ref" / "nn" / "gpt2"
    if not (ref_dir / "modules.py").exists():
        return None
    sys.path.insert(0, str(ROOT / "baseline"))
    from run_ref import build_reference_step

    return build_reference_step(ref_dir, MODEL, MICRO_B, SEQ, TOTAL_TOKENS, rank, world, local)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    if not torch.cuda.is_available():
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device on this machine"}))
            return
        raise SystemExit("bench.py needs a CUDA device")

    rank, world, local = dist_setup(args.gpus)
    try:
        built = build_ours(rank, world, local) if args.impl == "ours" else build_reference(rank, world, local)
    except Exception as e:  # the reference arm must never take the run down
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}))
            return
        raise
    if built is None:
        if rank == 0:
            print(json.dumps({"impl": "reference",
                              "unavailable": "baseline/_ref is missing (reference not installed)"}))
        return
    step, micro, launches_fn, path_name = built

    vocab = 50257
    host_batches = make_host_batches(micro, 1234 + rank, vocab)
    dev_batches = [(x.cuda(non_blocking=True), y.cuda(non_blocking=True)) for x, y in host_batches]
    torch.cuda.synchronize()

    # ---- device-timed, batches resident on the GPU
    for _ in range(args.warmup):
        step(dev_batches, False)
    barrier_sync(world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.perf_counter()
    ev0.record()
    for _ in range(args.steps):
        step(dev_batches, False)
    ev1.record()
    barrier_sync(world)
    dev_ms = max_over_ranks(ev0.elapsed_time(ev1), world) / args.steps

    # ---- end to end: pinned host -> device copies every micro-step, loss read every step
    for _ in range(2):
        step(host_batches, True)
    barrier_sync(world)
    t0 = time.perf_counter()
    last_loss = None
    for _ in range(args.steps):
        last_loss = step(host_batches, True)
    barrier_sync(world)
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, world) / args.steps
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        tokens = TOTAL_TOKENS
        h2d = sum(x.numel() * x.element_size() + y.numel() * y.element_size() for x, y in host_batches)
        out = {
            "metric": "GPT-2 124M train tokens/sec",
            "value": tokens / (dev_ms / 1e3),
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": dev_ms,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic (seeded uniform tokens, random-init weights)",
            "impl": args.impl,
            "config": {
                "model": "gpt2-124m (12L/12H/768, ctx 1024, vocab 50304, tied head, dropout 0)",
                "global_batch": tokens, "micro_batch": MICRO_B, "seq_len": SEQ,
                "micro_steps_per_rank": micro, "parallelism": f"dp{world}",
                "optimizer": "AdamW(0.9,0.95) wd 0.1 clip 1.0 lr 6e-4 cosine",
                "path": path_name,
                "l2": "inputs larger than L2 (activations of one micro-step are several GB)",
                "timing": "CUDA events on the launching stream, max over ranks",
            },
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "last_loss": last_loss},
            "gpu_launches": int(launches_fn()) * args.steps,
            "clocks": clocks,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
