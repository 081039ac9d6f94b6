"""Headline benchmark: GPT-2 training tokens/sec on N B200s of one node.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference model + torch DDP stack
    python bench.py --config 350m|1.5b ...    # the larger benchmark configurations (default 124m)

One step = one optimizer step over the configuration's total batch (124M: 524,288 tokens in
micro-batches of 16 x 1024 per rank), accumulated over micro-steps, then grad-norm clip + AdamW.
Tokens are seeded uniform integers, weights are random-init, dropout is 0 on both arms.

Two timings are taken, each over exactly `--steps` steps after `--warmup` untimed ones, with a
barrier + device synchronize on both sides and the max over ranks:
  * `value`     device time (CUDA events) with the token batches already resident on the GPU;
  * `e2e.value` through the public API with every micro-batch copied from pinned host memory
                and the step's loss read back to the host every step.
On more than one GPU a third timing gives `exposed_comm_ms`: the device-timed step minus the same
step (same micro-steps per rank) with the communicator replaced by the local optimizer, max over
ranks: what the cross-rank reduction, the sharded update and the parameter all-gather cost beyond
the compute they replace and overlap.
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

CONFIGS = {
    # name: (preset, model description, model kwargs, micro batch, total batch tokens)
    "124m": ("gpt2-124m", "gpt2-124m (12L/12H/768, ctx 1024, vocab 50304, tied head, dropout 0)",
             dict(vocab_size=50304, block_size=1024, emb_dim=768, num_heads=12, num_layers=12), 16, 524_288),
    "350m": ("gpt2-350m", "gpt2-350m (24L/16H/1024, ctx 1024, vocab 50304, tied head, dropout 0)",
             dict(vocab_size=50304, block_size=1024, emb_dim=1024, num_heads=16, num_layers=24), 8, 524_288),
    "1.5b": ("gpt2-1.5b", "gpt2-1.5b (48L/25H/1600, ctx 1024, vocab 50304, tied head, dropout 0)",
             dict(vocab_size=50304, block_size=1024, emb_dim=1600, num_heads=25, num_layers=48), 8, 1_048_576),
}
SEQ = 1024


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


def make_host_batches(n: int, seed: int, vocab: int, micro_b: int):
    """n pinned (X, Y) micro-batches of seeded uniform tokens, Y = X shifted by one."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        tok = torch.randint(0, vocab, (micro_b * SEQ + 1,), generator=g, dtype=torch.int64)
        out.append((tok[:-1].view(micro_b, SEQ).contiguous().pin_memory(),
                    tok[1:].view(micro_b, SEQ).contiguous().pin_memory()))
    return out


# ---------------------------------------------------------------------------------------------
# arm 1: this framework
# ---------------------------------------------------------------------------------------------
def build_ours(rank, world, local, conf, with_comm: bool = True):
    """Returns (step fn, micro-steps per rank, launches-per-step fn, path name, status check fn)."""
    from zero_to_hero_b200.config import get_preset
    from zero_to_hero_b200.engine import GPT2TrainEngine
    from zero_to_hero_b200.ops import _lib

    preset, _, model_kw, micro_b, total_tokens = conf
    cfg = get_preset(preset)
    for k, v in model_kw.items():
        setattr(cfg.model, k, v)
    cfg.train.micro_batch = micro_b
    cfg.train.total_batch_tokens = total_tokens
    if "Z2H_OVERLAP" in os.environ:  # A/B switch for the two-stream backward schedule
        cfg.train.overlap_wgrad = os.environ["Z2H_OVERLAP"] == "1"
    comm = None
    if world > 1 and with_comm:
        from zero_to_hero_b200.parallel.fused_ddp import FusedDDP
        # Z2H_NVLS=1 selects the multimem flavour; Z2H_BUCKET_MB overrides the bucket size (0 = one
        # reduction after backward)
        comm = FusedDDP(torch.device("cuda", local), nvls=os.environ.get("Z2H_NVLS", "0") == "1",
                        bucket_mb=float(os.environ.get("Z2H_BUCKET_MB", cfg.dist.bucket_mb)))
    eng = GPT2TrainEngine(cfg, device=torch.device("cuda", local), comm=comm)
    micro = max(1, total_tokens // (micro_b * SEQ * world))

    def step(batches, read_loss: bool):
        eng.train_step(batches)
        return eng.read_loss() if read_loss else None

    def check():
        _lib.check_status(torch.device("cuda", local))

    return step, micro, lambda: eng.kernel_launches_per_step(micro), "fused-engine", check


# ---------------------------------------------------------------------------------------------
# arm 2: the unmodified reference model driven as its DDP trainer drives it
# ---------------------------------------------------------------------------------------------
def build_reference(rank, world, local, conf):
    ref_dir = ROOT / "baseline" / "_ref" / "nn" / "gpt2"
    if not (ref_dir / "modules.py").exists():
        return None
    sys.path.insert(0, str(ROOT / "baseline"))
    from run_ref import build_reference_step

    _, _, model_kw, micro_b, total_tokens = conf
    out = build_reference_step(ref_dir, model_kw, micro_b, SEQ, total_tokens, rank, world, local)
    return (*out, lambda: None)


def timed_steps(step, batches, steps, world):
    """Device time per step (CUDA events on the launching stream), max over ranks."""
    barrier_sync(world)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        step(batches, False)
    ev1.record()
    barrier_sync(world)
    return max_over_ranks(ev0.elapsed_time(ev1), world) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="124m", choices=sorted(CONFIGS))
    ap.add_argument("--no-exposed-comm", action="store_true",
                    help="skip the compute-only third timing on multi-GPU runs")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    conf = CONFIGS[args.config]
    _, model_name, _, micro_b, total_tokens = conf

    if not torch.cuda.is_available():
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device on this machine"}))
            return
        raise SystemExit("bench.py needs a CUDA device")

    rank, world, local = dist_setup(args.gpus)
    try:
        built = (build_ours(rank, world, local, conf) if args.impl == "ours"
                 else build_reference(rank, world, local, conf))
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
    step, micro, launches_fn, path_name, check_status = built

    vocab = 50257
    host_batches = make_host_batches(micro, 1234 + rank, vocab, micro_b)
    dev_batches = [(x.cuda(non_blocking=True), y.cuda(non_blocking=True)) for x, y in host_batches]
    torch.cuda.synchronize()

    # ---- device-timed, batches resident on the GPU
    for _ in range(args.warmup):
        step(dev_batches, False)
    barrier_sync(world)
    check_status()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    dev_ms = timed_steps(step, dev_batches, args.steps, world)
    check_status()  # a bounded device wait that gave up would invalidate the number

    # ---- end to end: pinned host -> device copies every micro-step, loss read every step
    for _ in range(2):
        step(host_batches, True)
    barrier_sync(world)
    t0 = time.perf_counter()
    last_loss = None
    for _ in range(args.steps):
        last_loss = step(host_batches, True)  # reads the status word together with the loss
    barrier_sync(world)
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, world) / args.steps
    clocks = sampler.stop() if rank == 0 else None

    # ---- exposed communication: the same per-rank work with the local optimizer instead
    exposed = None
    gpu_launches = int(launches_fn()) * args.steps
    if world > 1 and args.impl == "ours" and not args.no_exposed_comm:
        del step, built, launches_fn, check_status  # the closures hold the first engine
        torch.cuda.empty_cache()
        local_step, _, _, _, local_check = build_ours(rank, world, local, conf, with_comm=False)
        for _ in range(args.warmup):
            local_step(dev_batches, False)
        compute_ms = timed_steps(local_step, dev_batches, args.steps, world)
        local_check()
        exposed = {"exposed_comm_ms": dev_ms - compute_ms, "compute_only_ms_per_step": compute_ms,
                   "how": "device-timed step minus the same micro-steps with the single-GPU optimizer "
                          "(no reduction, no sharding), both max over ranks"}

    if rank == 0:
        tokens = total_tokens
        h2d = sum(x.numel() * x.element_size() + y.numel() * y.element_size() for x, y in host_batches)
        out = {
            "metric": f"GPT-2 {args.config.upper()} train tokens/sec",
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
            "path": path_name,
            "config": {
                "model": model_name,
                "global_batch": tokens, "micro_batch": micro_b, "seq_len": SEQ,
                "micro_steps_per_rank": micro, "parallelism": f"dp{world}",
                "optimizer": "AdamW(0.9,0.95) wd 0.1 clip 1.0 lr 6e-4 cosine",
                "l2": "inputs larger than L2 (activations of one micro-step are several GB)",
                "timing": "CUDA events on the launching stream, max over ranks",
            },
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8 if args.impl == "ours" else 4,
                    "last_loss": last_loss},
            "gpu_launches": gpu_launches,
            "clocks": clocks,
        }
        if exposed is not None:
            out.update(exposed)
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
