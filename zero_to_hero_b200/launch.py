"""Job launcher: one training process per GPU of this node (or N CPU ranks over gloo).

    python -m zero_to_hero_b200.launch --gpus 8 -- --preset gpt2-124m train.steps=1000
    python -m zero_to_hero_b200.launch --ranks 2 --cpu -- --preset gpt2-tiny train.dtype=fp32 train.steps=3

The reference starts its trainers on rented machines through a Modal app (nn/gpt2/runner.py:22-54:
one function for `python train.py`, one that runs `torchrun --nproc-per-node 8 train_ddp.py`). Here
the same job is started on the local node: the launcher picks a free rendezvous port on 127.0.0.1,
exports RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT, starts `python -m
zero_to_hero_b200.train <args>` once per rank, streams rank 0's output, and ends the whole job with
a non-zero exit code as soon as one rank fails or the time limit passes (a rank that dies must not
leave the others waiting in a collective).
"""
from __future__ import annotations

import argparse
import os
import socket
import subprocess
import sys
import time


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(train_args: list[str], ranks: int, cpu: bool = False, timeout_s: float = 0.0,
           module: str = "zero_to_hero_b200.train") -> int:
    """Runs the job; returns its exit code (0 only if every rank exited 0)."""
    port = free_port()
    procs = []
    for r in range(ranks):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(ranks),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        if cpu:
            env["CUDA_VISIBLE_DEVICES"] = ""
        out = None if r == 0 else subprocess.DEVNULL
        procs.append(subprocess.Popen([sys.executable, "-m", module, *train_args], env=env, stdout=out,
                                      stderr=None if r == 0 else subprocess.STDOUT))
    t0 = time.time()
    code = 0
    try:
        while True:
            states = [p.poll() for p in procs]
            failed = [c for c in states if c not in (None, 0)]
            if failed:
                code = failed[0]
                break
            if all(c == 0 for c in states):
                break
            if timeout_s > 0 and time.time() - t0 > timeout_s:
                code = 124
                break
            time.sleep(0.2)
    finally:
        for p in procs:  # exactly the processes started here
            if p.poll() is None:
                p.terminate()
        for p in procs:
            try:
                p.wait(timeout=10)
            except subprocess.TimeoutExpired:
                p.kill()
    return code


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=0, help="ranks = GPUs of this node to use (0: all visible)")
    ap.add_argument("--ranks", type=int, default=0, help="number of ranks for --cpu")
    ap.add_argument("--cpu", action="store_true", help="CPU ranks over gloo (PyTorch module path)")
    ap.add_argument("--timeout", type=float, default=0.0, help="seconds; 0 = none")
    ap.add_argument("train_args", nargs=argparse.REMAINDER, help="arguments of zero_to_hero_b200.train after --")
    a = ap.parse_args()
    args = a.train_args[1:] if a.train_args[:1] == ["--"] else a.train_args
    if a.cpu:
        ranks = max(1, a.ranks)
    else:
        import torch

        ranks = a.gpus or torch.cuda.device_count()
        if ranks < 1:
            raise SystemExit("no GPU visible; use --cpu --ranks N")
    sys.exit(launch(args, ranks, cpu=a.cpu, timeout_s=a.timeout))


if __name__ == "__main__":
    main()
