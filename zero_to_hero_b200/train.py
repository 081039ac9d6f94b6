"""Training entry point.

    python -m zero_to_hero_b200.train --preset gpt2-124m train.steps=100
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m zero_to_hero_b200.train --preset gpt2-124m
    python -m zero_to_hero_b200.train --preset char-gpt train.data=char:path/to/input.txt

One code path covers the reference's single-GPU trainer (nn/gpt2/train.py), its DDP trainer
(nn/gpt2/train_ddp.py) and the char-level script (nn/gpt/3_gpt.py:152-248):
  * `train.dtype=bf16` on a GPU with a GPT-2 model runs the fused engine (hand-scheduled
    kernels, CUDA graph, fused peer-memory all-reduce + AdamW across ranks);
  * anything else (CPU, fp32, the char model) runs the PyTorch module path with
    torch AdamW (and torch DDP when launched with several ranks).
Adds what the reference lacks: gradient accumulation to `train.total_batch_tokens`, periodic
checkpoints, resume, JSONL logs, host-side failure detection between steps (heartbeats in the
job's key-value store; a rank that stops or leaves ends the job with exit code 3 instead of a
hang). Tokens/sec is device-timed (CUDA events) per logging window. Validation loss is a
forward-only pass (dropout off) and, with `train.hellaswag=<file.jsonl>`, HellaSwag accuracy is
scored through the same forward, strided over ranks and summed with two all-reduces, as the
reference does (nn/gpt2/train_ddp.py:110-121,152-157).
"""
from __future__ import annotations

import argparse
import os
import time

import torch
import torch.distributed as dist

from datetime import timedelta

from .config import Config, apply_overrides, get_preset
from .data.synthetic import SyntheticLoader
from .optim.adamw import build_optimizer, set_lr
from .optim.schedule import lr_for
from .utils.logging import StepLogger


def _dist_init(cfg: Config):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        backend = cfg.dist.backend if cfg.dist.backend != "auto" else ("nccl" if use_cuda else "gloo")
        kw = {"device_id": torch.device("cuda", local)} if backend == "nccl" else {}
        dist.init_process_group(backend, timeout=timedelta(seconds=cfg.dist.timeout_s), **kw)
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    return rank, world, device


def make_loaders(cfg: Config, device, rank, world):
    mc, tc = cfg.model, cfg.train
    if tc.data.startswith("char:"):
        from .data.text import CharTextLoader
        ld = CharTextLoader(tc.data[5:], tc.micro_batch, mc.block_size, "cpu", seed=tc.seed + rank)
        mc.vocab_size = ld.vocab.size
        return (lambda: ld.get_batch("train")), (lambda: ld.get_batch("val")), ld
    if tc.data.startswith("tokens:"):
        from .data.text import TokenFileLoader
        pin = device.type == "cuda"
        # the tail of the file is held out for validation and, like the reference's validation
        # loader (nn/gpt2/train_ddp.py:77), is not sharded by rank
        ld = TokenFileLoader(tc.data[7:], tc.micro_batch, mc.block_size, rank, world, pin=pin,
                             split="train", val_frac=tc.val_frac)
        va = TokenFileLoader(tc.data[7:], tc.micro_batch, mc.block_size, 0, 1, pin=pin,
                             split="val", val_frac=tc.val_frac)
        return ld.next_host_batch, va.next_host_batch, ld
    real_vocab = min(mc.vocab_size, 50257) if mc.vocab_size >= 50257 else mc.vocab_size
    tr = SyntheticLoader("train", tc.micro_batch, mc.block_size, real_vocab, device, rank, world, tc.seed)
    va = SyntheticLoader("val", tc.micro_batch, mc.block_size, real_vocab, device, 0, 1, tc.seed)
    return tr.next_host_batch, va.next_host_batch, tr


def train(cfg: Config, resume: str = "") -> dict:
    rank, world, device = _dist_init(cfg)
    master = rank == 0
    torch.manual_seed(cfg.train.seed)
    if device.type == "cuda":
        torch.set_float32_matmul_precision("high")
    next_train, next_val, loader = make_loaders(cfg, device, rank, world)
    mc, tc, oc = cfg.model, cfg.train, cfg.optim
    tokens_per_micro = tc.micro_batch * mc.block_size * world
    accum = max(1, tc.total_batch_tokens // tokens_per_micro)
    fused = (device.type == "cuda" and tc.dtype == "bf16" and mc.kind == "gpt2" and mc.head_dim == 64)
    logger = StepLogger(tc.log_jsonl, master)
    if master:
        print(cfg.to_json())
        print(f"path: {'fused engine' if fused else 'pytorch modules'} | world {world} | "
              f"micro-steps per step {accum}")
    history = []

    if fused:
        from .engine import GPT2TrainEngine, load_engine_checkpoint, save_engine_checkpoint
        from .parallel.health import HeartbeatMonitor, default_store
        comm = None
        monitor = None
        if world > 1:
            from .parallel.fused_ddp import FusedDDP, TorchDDPComm
            if cfg.dist.fused_allreduce:
                comm = FusedDDP(device, budget_s=cfg.dist.device_wait_s, nvls=cfg.dist.nvls,
                                bucket_mb=cfg.dist.bucket_mb)
            else:
                comm = TorchDDPComm(device)
            if cfg.dist.heartbeat_interval > 0:
                monitor = HeartbeatMonitor(default_store(), rank, world, timeout_s=cfg.dist.timeout_s)
        eng = GPT2TrainEngine(cfg, device, comm=comm)
        start = 0
        if resume:
            ck = load_engine_checkpoint(eng, resume, elastic=tc.elastic_resume)
            start = int(ck["step"])
            if ck.get("data") and hasattr(loader, "load_state"):
                loader.load_state(ck["data"])  # this rank's own cursor / generator state
        if master:
            print(f"num_params: {eng.layout.num_params():,}")
        examples = None
        if tc.hellaswag:
            from .eval.hellaswag import load_examples
            examples = load_examples(tc.hellaswag)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        window = 0
        for step in range(start, tc.steps):
            if monitor is not None and step % cfg.dist.heartbeat_interval == 0:
                # every peer's host has reached this step, so the fused kernels launched below
                # only ever wait for step skew; a peer that stopped raises RankFailure here,
                # before any kernel that would wait for it is launched
                monitor.beat(step)
                monitor.wait_all(step)
            lr = lr_for(step, oc)
            eng.train_step([next_train() for _ in range(accum)], lr)
            window += 1
            if step % tc.log_interval == 0 or step == tc.steps - 1:
                ev1.record()
                loss = eng.read_loss()  # also raises if a device-side wait gave up
                ms = ev0.elapsed_time(ev1) / max(window, 1)
                rec = dict(train=loss, grad_norm=eng.read_grad_norm(), lr=lr, ms=ms,
                           tok_s=tokens_per_micro * accum / (ms / 1e3))
                if world > 1:
                    t = torch.tensor([loss, ms], device=device, dtype=torch.float64)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    rec["ms_max_over_ranks"] = float(t[1])
                    rec["tok_s"] = tokens_per_micro * accum / (float(t[1]) / 1e3)
                    rec["ms_rank"] = ms
                if tc.eval_interval and step % tc.eval_interval == 0:
                    rec["val"] = evaluate_engine(eng, next_val, tc.eval_batches, world)
                    if examples is not None:
                        rec["hellaswag"] = hellaswag_engine(eng, examples, rank, world)
                logger.log(step, **rec)
                history.append({"step": step, **rec})
                ev0.record()
                window = 0
            if tc.checkpoint_dir and tc.checkpoint_interval and (step + 1) % tc.checkpoint_interval == 0:
                st = loader.state() if hasattr(loader, "state") else None
                save_engine_checkpoint(eng, os.path.join(tc.checkpoint_dir, f"step{step + 1:08d}.pt"), st)
        result = {"history": history, "engine": eng}
    else:
        result = _train_modules(cfg, device, rank, world, accum, next_train, next_val, loader, logger,
                                resume, history)
    logger.close()
    return result


def evaluate_engine(eng, next_val, batches: int, world: int) -> float:
    """Validation loss through the engine's forward-only path: dropout off, no backward, own CUDA
    graph; gradients, dropout seed and micro-step counter of the training run are untouched."""
    total = 0.0
    for _ in range(batches):
        total += eng.eval_loss(*next_val())
    loss = total / batches
    if world > 1:
        t = torch.tensor([loss], device=eng.device)
        dist.all_reduce(t, op=dist.ReduceOp.AVG)
        loss = float(t.item())
    return loss


def hellaswag_engine(eng, examples, rank: int, world: int) -> float:
    """HellaSwag accuracy through the engine's forward; examples strided over ranks, `correct`
    and `total` summed with two all-reduces (nn/gpt2/train_ddp.py:152-157)."""
    from .eval.hellaswag import evaluate_losses_fn

    correct, total = evaluate_losses_fn(eng.eval_losses, examples, eng.device, eng.mc.block_size,
                                        rank, world)
    if world > 1:
        dist.all_reduce(correct, op=dist.ReduceOp.SUM)
        dist.all_reduce(total, op=dist.ReduceOp.SUM)
    return float(correct.item()) / max(1, int(total.item()))


def build_module(cfg: Config):
    mc = cfg.model
    if mc.kind == "char":
        from .models.gpt import GPTLM
        return GPTLM(mc.vocab_size, mc.block_size, mc.emb_dim, mc.num_layers, mc.num_heads, mc.dropout)
    from .models.gpt2 import GPT2
    return GPT2(mc)


def _train_modules(cfg, device, rank, world, accum, next_train, next_val, loader, logger, resume, history):
    from .utils.checkpoint import load_checkpoint, save_checkpoint, set_rng_state
    mc, tc, oc = cfg.model, cfg.train, cfg.optim
    model = build_module(cfg).to(device)
    raw = model
    if world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP
        model = DDP(model, device_ids=[device.index] if device.type == "cuda" else None)
    opt = build_optimizer(raw, oc, device.type)
    start = 0
    if resume:
        ck = load_checkpoint(resume)
        raw.load_state_dict(ck["model"], strict=False)
        opt.load_state_dict(ck["optim"])
        start = int(ck["step"])
        set_rng_state(ck["rng"])
    if rank == 0:
        print(f"num_params: {sum(p.numel() for p in raw.parameters()):,}")
    model.train()
    t0 = time.perf_counter()
    for step in range(start, tc.steps):
        lr = lr_for(step, oc)
        set_lr(opt, lr)
        opt.zero_grad(set_to_none=True)
        loss_acc = 0.0
        for i in range(accum):
            X, Y = next_train()
            X, Y = X.to(device), Y.to(device)
            sync = (i == accum - 1) or world == 1
            ctx = model.no_sync() if (world > 1 and not sync) else _null()
            with ctx:
                _, loss = model(X, Y)
                (loss / accum).backward()
            loss_acc += float(loss.detach()) / accum
        gn = float(torch.nn.utils.clip_grad_norm_(raw.parameters(), oc.clip_norm)) if oc.clip_norm > 0 else 0.0
        opt.step()
        if step % tc.log_interval == 0 or step == tc.steps - 1:
            if device.type == "cuda":
                torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            rec = dict(train=loss_acc, grad_norm=gn, lr=lr, ms=dt * 1e3)
            if tc.eval_interval and step % tc.eval_interval == 0:
                model.eval()
                with torch.inference_mode():
                    vl = 0.0
                    for _ in range(tc.eval_batches):
                        X, Y = next_val()
                        vl += float(raw(X.to(device), Y.to(device))[1]) / tc.eval_batches
                    if tc.hellaswag:
                        from .eval.hellaswag import evaluate as hs_evaluate, load_examples
                        c, n = hs_evaluate(raw, load_examples(tc.hellaswag), device, mc.block_size,
                                           rank, world)
                        if world > 1:
                            dist.all_reduce(c, op=dist.ReduceOp.SUM)
                            dist.all_reduce(n, op=dist.ReduceOp.SUM)
                        rec["hellaswag"] = float(c.item()) / max(1, int(n.item()))
                model.train()
                rec["val"] = vl
            logger.log(step, **rec)
            history.append({"step": step, **rec})
            t0 = time.perf_counter()
        if tc.checkpoint_dir and tc.checkpoint_interval and (step + 1) % tc.checkpoint_interval == 0 and rank == 0:
            save_checkpoint(os.path.join(tc.checkpoint_dir, f"step{step + 1:08d}.pt"), raw.state_dict(),
                            opt.state_dict(), step + 1, None, cfg.to_dict())
    return {"history": history, "model": raw}


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="gpt2-124m")
    ap.add_argument("--resume", default="")
    ap.add_argument("overrides", nargs="*", help="section.key=value")
    a = ap.parse_args(argv)
    cfg = apply_overrides(get_preset(a.preset), a.overrides)
    from .parallel.health import RankFailure
    try:
        train(cfg, a.resume)
    except RankFailure as e:
        # a peer stopped between steps: nothing of ours is in flight towards it, so leave at once
        # with a code the launcher turns into the job's exit code
        print(f"[rank {os.environ.get('RANK', '0')}] stopping: {e}", flush=True)
        os._exit(3)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
