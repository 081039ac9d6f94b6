"""Micro-benchmarks of single kernels with CUDA-event timing and roofline fractions.

    python -m zero_to_hero_b200.utils.kernel_bench --kernel gemm --M 16384 --N 2304 --K 768
    python -m zero_to_hero_b200.utils.kernel_bench --kernel flash_fwd --B 16 --T 1024 --H 12
    python -m zero_to_hero_b200.utils.kernel_bench --kernel all

Timing hygiene: >= 3 warm-up launches, events on the launching stream, and an L2 flush (a
256 MiB memset) between timed launches unless --no-flush. Peaks come from MEASURED_PEAKS.json
at the repository root when present (else 6.65 TB/s and 1590 TFLOP/s, marked "of fallback").
The reference's counterparts are the `Bench` harnesses inside its puzzles
(gpu-mojo/problems/p23/p23.mojo:474-529, p24/p24.mojo:425-511, p30/p30.mojo:381-403).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from ..ops import _lib, gemm as G, native as N


def peaks() -> tuple[float, float, str]:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


_flush_buf = None


def flush_l2():
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_kernel(fn, iters: int, warmup: int = 3, flush: bool = True) -> float:
    """Median milliseconds of one call of fn()."""
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        if flush:
            # three passes keep the GPU busy for ~130 us, so the host has queued the events and the
            # launch before the GPU reaches them and no launch latency falls between the events
            for _ in range(3):
                flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def report(name: str, ms: float, flops: float = 0.0, bytes_: float = 0.0) -> dict:
    hbm, tf, tag = peaks()
    out = {"kernel": name, "ms": round(ms, 5)}
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out["frac_tensor"] = f"{flops / ms / 1e9 / tf:.3f} {tag}"
    if bytes_:
        out["gbs"] = round(bytes_ / ms / 1e6, 1)
        out["frac_hbm"] = f"{bytes_ / ms / 1e6 / hbm:.3f} {tag}"
    print(json.dumps(out), flush=True)
    return out


def bench_gemm(a, dev):
    M, Nn, K = a.M, a.N, a.K
    A = torch.randn((K, M) if a.a_mn else (M, K), device=dev).bfloat16()
    B = torch.randn((K, Nn) if a.b_mn else (Nn, K), device=dev).bfloat16()
    out = torch.zeros(M, Nn, device=dev, dtype=torch.float32 if a.fp32_out else torch.bfloat16)
    kw = {}
    if a.split_k > 1 or a.split_k == 0:  # 0: stream-K schedule
        kw = dict(epi=G.EPI_ATOMIC_ADD, split_k=a.split_k)
    tag = ""
    if a.epi != "none":  # the fused epilogues of the MLP and the projections (bf16 output)
        other = torch.randn(M, Nn, device=dev).bfloat16()
        bias = torch.randn(Nn, device=dev).bfloat16()
        kw = {"bias": dict(bias=bias),
              "gelu": dict(bias=bias, aux_out=other, epi=G.EPI_GELU),
              "gelu_grad": dict(aux_in=other, epi=G.EPI_GELU_GRAD),
              "gelu_save_grad": dict(bias=bias, aux_out=other, epi=G.EPI_GELU_SAVE_GRAD),
              "mul_aux": dict(aux_in=other, epi=G.EPI_MUL_AUX),
              "residual": dict(bias=bias, residual=other, epi=G.EPI_RESIDUAL)}[a.epi]
        if a.colsum:
            kw["colsum"] = torch.zeros(Nn, device=dev)
        tag = f" epi={a.epi}{'+colsum' if a.colsum else ''}"
    ms = time_kernel(lambda: G.gemm(A, B, out, a_mn=a.a_mn, b_mn=a.b_mn, **kw), a.iters, flush=not a.no_flush)
    report(f"gemm M{M} N{Nn} K{K} a_mn{int(a.a_mn)} b_mn{int(a.b_mn)} split{a.split_k}{tag}", ms,
           flops=2.0 * M * Nn * K)
    if a.compare and not (a.a_mn or a.b_mn):
        ms2 = time_kernel(lambda: torch.matmul(A, B.t()), a.iters, flush=not a.no_flush)
        report("  torch.matmul (cuBLAS) same shape", ms2, flops=2.0 * M * Nn * K)


def bench_flash(a, dev, which):
    B, T, H = a.B, a.T, a.H
    C = H * 64
    qkv = (torch.randn(B * T, 3 * C, device=dev) * 0.7).bfloat16()
    out = torch.empty(B * T, C, device=dev, dtype=torch.bfloat16)
    lse = torch.empty(B, H, T, device=dev)
    fl = 4.0 * B * H * T * T * 64 / 2
    N.flash_fwd(qkv, out, lse, B, T, H)
    if which == "flash_fwd":
        ms = time_kernel(lambda: N.flash_fwd(qkv, out, lse, B, T, H), a.iters, flush=not a.no_flush)
        report(f"flash_fwd B{B} T{T} H{H}", ms, flops=fl)
    else:
        dout = torch.randn_like(out)
        dqkv = torch.empty_like(qkv)
        dqa = torch.empty(N.flash_bwd_dq_elems(B, T, H), device=dev)
        stats = torch.empty(N.flash_bwd_stats_elems(B, T, H), device=dev)
        ms = time_kernel(lambda: N.flash_bwd(qkv, out, dout, lse, dqkv, dqa, stats, B, T, H), a.iters,
                         flush=not a.no_flush)
        report(f"flash_bwd B{B} T{T} H{H} (3 launches)", ms, flops=2.5 * fl)
    if a.compare:
        import torch.nn.functional as F
        q, k, v = [x.reshape(B, T, H, 64).transpose(1, 2) for x in qkv.split(C, dim=1)]
        if which == "flash_fwd":
            ms2 = time_kernel(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True), a.iters,
                              flush=not a.no_flush)
            report("  torch SDPA forward same shape", ms2, flops=fl)
        else:
            qq, kk, vv = [x.detach().requires_grad_(True) for x in (q, k, v)]
            o = F.scaled_dot_product_attention(qq, kk, vv, is_causal=True)
            g = torch.randn_like(o)
            ms2 = time_kernel(lambda: torch.autograd.grad(o, (qq, kk, vv), g, retain_graph=True), a.iters,
                              flush=not a.no_flush)
            report("  torch SDPA backward same shape", ms2, flops=2.5 * fl)


def bench_layernorm(a, dev):
    M, C = a.M, a.C
    x = torch.randn(M, C, device=dev).bfloat16()
    w = torch.ones(C, device=dev).bfloat16()
    y = torch.empty_like(x)
    mean, rstd = torch.empty(M, device=dev), torch.empty(M, device=dev)
    ms = time_kernel(lambda: N.layernorm_fwd(x, w, None, y, mean, rstd), a.iters, flush=not a.no_flush)
    report(f"layernorm_fwd M{M} C{C}", ms, bytes_=2.0 * M * C * 2)
    dy = torch.randn_like(x)
    dx = torch.empty_like(x)
    dw = torch.zeros(C, device=dev)
    scratch = torch.empty(N.layernorm_bwd_num_partials(M) * 2 * C, device=dev)
    ms = time_kernel(lambda: N.layernorm_bwd(dy, x, w, mean, rstd, dy, dx, dw, None, scratch), a.iters,
                     flush=not a.no_flush)
    report(f"layernorm_bwd M{M} C{C} (2 launches)", ms, bytes_=4.0 * M * C * 2)


def bench_ce(a, dev):
    M, V = a.M, a.V
    logits = torch.randn(M, V, device=dev).bfloat16()
    tg = torch.randint(0, V, (M,), device=dev)
    losses = torch.empty(M, device=dev)
    ms = time_kernel(lambda: N.ce_fwd_bwd(logits, tg, losses, V, 1.0 / M), a.iters, flush=not a.no_flush)
    report(f"ce_fwd_bwd M{M} V{V}", ms, bytes_=2.0 * M * V * 2)


def bench_adamw(a, dev):
    n = a.n
    p, g, m, v = (torch.randn(n, device=dev) * 0.01 for _ in range(4))
    v = v.abs()
    p16 = torch.empty(n, device=dev, dtype=torch.bfloat16)
    hyper = torch.tensor([6e-4, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0, 1.0] + [0] * 7, device=dev)
    partials = torch.empty(1024, device=dev)
    norm = torch.zeros(1, device=dev)

    def run():
        k = N.gradnorm_partials(g, partials)
        N.adamw_step(p, g, m, v, p16, n // 2, hyper, partials, k, norm, zero_grad=False)

    ms = time_kernel(run, a.iters, flush=not a.no_flush)
    report(f"gradnorm + adamw n{n} (2 launches)", ms, bytes_=n * (4 * 5 + 4 * 3 + 2.0))


def bench_embedding(a, dev):
    M, C, V, T = a.M, a.C, a.V, a.T
    idx = torch.randint(0, V, (M,), device=dev)
    wte = torch.randn(V, C, device=dev).bfloat16()
    wpe = torch.randn(T, C, device=dev).bfloat16()
    out = torch.empty(M, C, device=dev, dtype=torch.bfloat16)
    ms = time_kernel(lambda: N.embed_fwd(idx.view(-1, T), wte, wpe, out, T), a.iters, flush=not a.no_flush)
    report(f"embed_fwd M{M} C{C} V{V}", ms, bytes_=2.0 * M * C * 2 + T * C * 2)
    dx = torch.randn(M, C, device=dev).bfloat16()
    dwte = torch.zeros(V, C, device=dev)
    dwpe = torch.zeros(T, C, device=dev)
    ms = time_kernel(lambda: N.embed_bwd(idx.view(-1, T), dx, dwte, dwpe, M // T, T), a.iters,
                     flush=not a.no_flush)
    # dx is read by both kernels; the scattered rows are read-modify-written in fp32
    report(f"embed_bwd M{M} C{C} (2 launches)", ms, bytes_=2.0 * M * C * 2 + 2.0 * M * C * 4 + 2.0 * T * C * 4)


def bench_dropout(a, dev):
    M, C = a.M, a.C
    x = torch.randn(M, C, device=dev).bfloat16()
    r = torch.randn(M, C, device=dev).bfloat16()
    out = torch.empty_like(x)
    seed = torch.tensor([1234], device=dev, dtype=torch.int64)
    ms = time_kernel(lambda: N.dropout_apply(x, out, 0.2, seed, 3, residual=r), a.iters, flush=not a.no_flush)
    report(f"dropout_apply (+residual) M{M} C{C}", ms, bytes_=3.0 * M * C * 2)


def bench_colsum(a, dev):
    M, Nn = a.M, a.N
    dy = torch.randn(M, Nn, device=dev).bfloat16()
    db = torch.zeros(Nn, device=dev)
    ms = time_kernel(lambda: N.colsum_bf16(dy, db), a.iters, flush=not a.no_flush)
    report(f"colsum_bf16 M{M} N{Nn}", ms, bytes_=1.0 * M * Nn * 2)


def bench_sample(a, dev):
    from ..ops.sampling import sample_topk_native
    B, V = a.B, a.V
    logits = torch.randn(B, V, device=dev)
    ms = time_kernel(lambda: sample_topk_native(logits, 0.8, 50, 7, 0), a.iters, flush=not a.no_flush)
    report(f"sample_topk B{B} V{V} top-k 50", ms, bytes_=1.0 * B * V * 4)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all")
    ap.add_argument("--epi", default="none", choices=["none", "bias", "gelu", "gelu_grad", "gelu_save_grad", "mul_aux", "residual"],
                    help="gemm: fused epilogue to time")
    ap.add_argument("--colsum", action="store_true", help="gemm: also produce the column sums of the output")
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=2304)
    ap.add_argument("--K", type=int, default=768)
    ap.add_argument("--C", type=int, default=768)
    ap.add_argument("--V", type=int, default=50304)
    ap.add_argument("--B", type=int, default=16)
    ap.add_argument("--T", type=int, default=1024)
    ap.add_argument("--H", type=int, default=12)
    ap.add_argument("--n", type=int, default=124_000_000)
    ap.add_argument("--a-mn", dest="a_mn", action="store_true")
    ap.add_argument("--b-mn", dest="b_mn", action="store_true")
    ap.add_argument("--fp32-out", dest="fp32_out", action="store_true")
    ap.add_argument("--split-k", dest="split_k", type=int, default=1,
                    help="> 1: split-K slices, 0: stream-K (both with fp32 atomic accumulation)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--compare", action="store_true", help="also time the PyTorch library op")
    ap.add_argument("--gemm-algo", dest="gemm_algo", type=int, default=-1,
                    help="0: one-CTA kernel, 1: CTA-pair kernel wherever it applies, 2: automatic")
    a = ap.parse_args()
    if a.gemm_algo >= 0:
        G.set_algo(a.gemm_algo)
    if a.split_k != 1:
        a.fp32_out = True
    dev = torch.device("cuda")
    torch.manual_seed(0)
    k = a.kernel
    if k in ("gemm", "all"):
        if k == "all":
            for (M, Nn, K) in [(16384, 2304, 768), (16384, 768, 768), (16384, 3072, 768),
                               (16384, 768, 3072), (16384, 50304, 768), (8192, 8192, 8192)]:
                a.M, a.N, a.K = M, Nn, K
                bench_gemm(a, dev)
        else:
            bench_gemm(a, dev)
    if k in ("flash_fwd", "all"):
        bench_flash(a, dev, "flash_fwd")
    if k in ("flash_bwd", "all"):
        bench_flash(a, dev, "flash_bwd")
    if k in ("layernorm", "all"):
        a.M = 16384 if k == "all" else a.M
        bench_layernorm(a, dev)
    if k in ("ce", "all"):
        a.M = 16384 if k == "all" else a.M
        bench_ce(a, dev)
    if k in ("adamw", "all"):
        bench_adamw(a, dev)
    if k in ("embedding", "all"):
        a.M = 16384 if k == "all" else a.M
        bench_embedding(a, dev)
    if k in ("dropout", "all"):
        bench_dropout(a, dev)
    if k in ("colsum", "all"):
        a.N = 3072 if k == "all" else a.N
        bench_colsum(a, dev)
    if k in ("sample", "all"):
        bench_sample(a, dev)
    torch.cuda.synchronize()
    _lib.check_status()


if __name__ == "__main__":
    main()
