"""All-reduce and fused all-reduce + AdamW size sweep over NVLink peer memory, against NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m zero_to_hero_b200.parallel.allreduce_bench [--min-bytes 1024] [--max-bytes 1073741824]

For every size (powers of `--step`, default 4, between the bounds) and dtype (fp32, bf16) it
times, on the device with CUDA events and as the maximum over ranks:
  * this package's one-shot and two-shot all-reduce kernels (plain peer loads / stores) and,
    where the system provides a multicast address, the one-kernel multimem (NVLS) all-reduce,
  * NCCL's all-reduce through torch.distributed,
and, for the fp32 sizes, the whole optimizer step of a flat parameter vector of that many
gradients:
  * fused: reduce + clip + AdamW + bf16 weights on every rank (`FusedDDP.fused_step`, no library
    call) in its two-shot form (each rank owns 1/world, peer loads / stores or multimem) and, up
    to 16 MiB, in its one-shot form (every rank reduces everything, replicated state, no
    all-gather): the crossover between the two is what `FusedDDP(one_shot_kb=...)` encodes,
  * baseline: NCCL all-reduce followed by the single-GPU norm + AdamW kernels on every rank.
Bus bandwidth is the usual 2 (n-1)/n * bytes / time; `frac_of_900` and `frac_of_770` relate it to
the nominal NVLink rate per direction per GPU and to the measured peer-copy rate (for the peer
load / store algorithms 2 (n-1)/n * bytes is what has to arrive at every GPU). One JSON line per
measurement on rank 0.
The waits inside the kernels are bounded; a rank that does not show up ends them with a status
code instead of a hang.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import native as N
from .fused_ddp import NVLS, ONE_SHOT, TWO_SHOT, FusedDDP, PeerComm, SymmetricBuffer


def _time(fn, iters: int, warmup: int, group) -> float:
    """Milliseconds per call, maximum over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=1 << 10)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--step", type=int, default=4, help="ratio between consecutive sizes (2 or 4)")
    ap.add_argument("--skip-optimizer", action="store_true")
    ap.add_argument("--skip-allreduce", action="store_true")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    comm = PeerComm(dev)
    bus = 2.0 * (world - 1) / world

    def emit(**kw):
        if rank == 0:
            print(json.dumps(kw), flush=True)

    sizes = []
    b = a.min_bytes
    while b <= a.max_bytes:
        sizes.append(b)
        b *= a.step

    def bw(nbytes, ms):
        g = bus * nbytes / ms / 1e6
        return round(g, 1), round(g / 900.0, 3), round(g / 770.0, 3)

    for dtype in (() if a.skip_allreduce else (torch.float32, torch.bfloat16)):
        for nbytes in sizes:
            n = max(8 * world, nbytes // dtype.itemsize // (8 * world) * (8 * world))
            buf = SymmetricBuffer(n, dtype, dev)
            buf.tensor.normal_()
            ref = buf.tensor.clone()
            out = torch.empty_like(buf.tensor)
            iters = a.iters if nbytes <= (16 << 20) else max(3, a.iters // 4)
            nb = n * dtype.itemsize
            res = {"op": "allreduce", "dtype": str(dtype).split(".")[-1], "bytes": nb, "world": world}
            if nbytes <= (8 << 20):  # one-shot reads every peer's full buffer: small sizes only
                ms = _time(lambda: comm.allreduce_(buf, out=out, algo=ONE_SHOT), iters, a.warmup, group)
                res["oneshot_us"] = round(ms * 1e3, 2)
                res["oneshot_busbw_gbs"], res["oneshot_frac_of_900"], _ = bw(nb, ms)
            ms = _time(lambda: comm.allreduce_(buf, algo=TWO_SHOT), iters, a.warmup, group)
            res["twoshot_us"] = round(ms * 1e3, 2)
            res["twoshot_busbw_gbs"], res["twoshot_frac_of_900"], res["twoshot_frac_of_770"] = bw(nb, ms)
            if buf.multicast_ptr:
                ms = _time(lambda: comm.allreduce_(buf, algo=NVLS), iters, a.warmup, group)
                res["nvls_us"] = round(ms * 1e3, 2)
                res["nvls_busbw_gbs"], res["nvls_frac_of_900"], res["nvls_frac_of_770"] = bw(nb, ms)
            ms = _time(lambda: dist.all_reduce(ref, group=group), iters, a.warmup, group)
            res["nccl_us"] = round(ms * 1e3, 2)
            res["nccl_busbw_gbs"], res["nccl_frac_of_900"], _ = bw(nb, ms)
            _lib.check_status(dev)
            emit(**res)
            del buf, ref, out
            torch.cuda.empty_cache()

    if not a.skip_optimizer:
        hyper = torch.tensor([1e-4, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0, 1.0], device=dev)
        norm = torch.zeros(1, device=dev)
        for nbytes in sizes:
            n = max(8 * world, nbytes // 4 // (8 * world) * (8 * world))
            iters = a.iters if nbytes <= (16 << 20) else max(3, a.iters // 4)
            ms_flavour = {}
            flavours = [("p2p", dict(nvls=False, one_shot_kb=0)), ("nvls", dict(nvls=True, one_shot_kb=0))]
            if nbytes <= (16 << 20):
                flavours.append(("oneshot", dict(nvls=False, one_shot_kb=1 << 20)))
            for name, kw in flavours:
                fused = FusedDDP(dev, bucket_mb=0, **kw)
                fused.setup(n, n)
                if kw["nvls"] and not fused.nvls:  # no multicast address on this system
                    del fused
                    continue
                fused.g.normal_(std=0.01)
                fused.load_master(torch.zeros(n, device=dev))
                ms_flavour[name] = _time(lambda: fused.fused_step(hyper, norm), iters, a.warmup, group)
                del fused
                torch.cuda.empty_cache()
            ms_f = ms_flavour["p2p"]
            # baseline: library all-reduce, then the single-GPU norm + AdamW kernels, replicated
            g = torch.randn(n, device=dev) * 0.01
            p32, m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
            p16 = torch.zeros(n, device=dev, dtype=torch.bfloat16)
            partials = torch.zeros(4096, device=dev)

            def baseline():
                dist.all_reduce(g, group=group)
                k = N.gradnorm_partials(g, partials)
                N.adamw_step(p32, g, m, v, p16, n, hyper, partials, k, norm, zero_grad=False)

            ms_b = _time(baseline, iters, a.warmup, group)
            _lib.check_status(dev)
            best = min(ms_flavour.values())
            # bytes that must arrive at every GPU in the two-shot form: its share of the fp32
            # gradients from the n-1 peers, then the other shards' bf16 weights
            link_bytes = (world - 1) / world * n * (4 + 2)
            emit(op="allreduce+adamw", grad_bytes=n * 4, world=world, fused_us=round(ms_f * 1e3, 2),
                 fused_nvls_us=round(ms_flavour["nvls"] * 1e3, 2) if "nvls" in ms_flavour else None,
                 fused_oneshot_us=round(ms_flavour["oneshot"] * 1e3, 2) if "oneshot" in ms_flavour else None,
                 nccl_plus_adamw_us=round(ms_b * 1e3, 2), speedup=round(ms_b / best, 3),
                 roofline_us_at_770=round(link_bytes / 770e9 * 1e6, 2),
                 frac_of_roofline=round(link_bytes / 770e9 * 1e3 / ms_f, 3))
            del g, p32, m, v, p16
            torch.cuda.empty_cache()
    dist.barrier(group)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
