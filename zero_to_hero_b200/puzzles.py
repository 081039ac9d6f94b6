"""Per-puzzle command line: runs a primitive on the shapes the reference's puzzle hard-codes and
checks the result against a CPU oracle, printing `out`, `expected` and a verdict.

    python -m zero_to_hero_b200.puzzles p01
    python -m zero_to_hero_b200.puzzles p16 --tiled
    python -m zero_to_hero_b200.puzzles p33 --tensor-core
    python -m zero_to_hero_b200.puzzles all
    python -m zero_to_hero_b200.puzzles p23 --benchmark     # also p24, p30, p31, p32

Counterpart of the reference's `pixi run pNN [-- --flag]` tasks (gpu-mojo/pixi.toml:60-129) and
the `main()` of every puzzle (e.g. gpu-mojo/problems/p16/p16.mojo:148-231). Flags select the
variant exactly as there; without a flag the first variant runs. `--benchmark` runs the size
sweeps of the reference's in-puzzle `Bench` harnesses (gpu-mojo/problems/p23/p23.mojo:474-529,
p24/p24.mojo:425-511, p30/p30.mojo:381-403, p31/p31.mojo:489-504, p32/p32.mojo) with CUDA-event
timing (3 warm-ups, median of 20, L2 flushed between launches) and prints one JSON line per
variant and size with microseconds and achieved GB/s.
"""
from __future__ import annotations

import argparse
import sys

import torch

from .ops import primitives as P


def _check(name, got, ref, tol=1e-5):
    got, ref = got.float().cpu(), torch.as_tensor(ref).float().cpu()
    ok = got.shape == ref.shape and torch.allclose(got, ref, atol=tol, rtol=tol)
    flat_g, flat_r = got.reshape(-1), ref.reshape(-1)
    print(f"[{name}] out: {flat_g[:8].tolist()}{' ...' if flat_g.numel() > 8 else ''}")
    print(f"[{name}] expected: {flat_r[:8].tolist()}{' ...' if flat_r.numel() > 8 else ''}")
    print(f"[{name}] {'PASS' if ok else 'FAIL'}")
    return ok


def cu(x):
    return torch.as_tensor(x, dtype=torch.float32).cuda()


def p01(f):
    a = torch.arange(4.0)
    return _check("p01 add_10", P.add10(cu(a), block=4), a + 10)


def p02(f):
    a, b = torch.arange(4.0), torch.arange(4.0)
    return _check("p02 add", P.zip_add(cu(a), cu(b), block=4), a + b)


def p03(f):
    a = torch.arange(4.0)
    return _check("p03 add_10_guard", P.add10(cu(a), block=8), a + 10)


def p04(f):
    a = torch.arange(4.0).view(2, 2)
    return _check("p04 add_10_2d", P.add10_2d(cu(a), block=(3, 3)), a + 10)


def p05(f):
    a, b = torch.arange(2.0), torch.arange(2.0)
    return _check("p05 broadcast_add", P.broadcast_add(cu(a), cu(b)), a[None, :] + b[:, None])


def p06(f):
    a = torch.arange(9.0)
    return _check("p06 add_10_blocks", P.add10(cu(a), block=4), a + 10)


def p07(f):
    a = torch.arange(25.0).view(5, 5)
    return _check("p07 add_10_blocks_2d", P.add10_2d(cu(a), block=(3, 3)), a + 10)


def p08(f):
    a = torch.ones(8)
    return _check("p08 add_10_shared", P.add10_shared(cu(a), block=4), a + 10)


def p09(f):
    a = torch.arange(4.0)
    if f == "third-case":
        return _check("p09 collaborative_filter", P.collaborative_filter(cu(a)), P.oracle_collaborative_filter(a))
    if f == "second-case":
        return _check("p09 sliding_window", P.sliding_window3(cu(a)), P.oracle_sliding_window3(a))
    return _check("p09 add_10", P.add10(cu(a), block=4), a + 10)


def p10(f):
    a = torch.arange(4.0).view(2, 2)
    ok = _check("p10 shared_sum (initialised accumulator)", P.shared_sum_broadcast(cu(a)), torch.full((2, 2), 6.0))
    out, bad, who, idx = P.checked_gather(cu(torch.arange(8.0)), torch.tensor([1, 9, 3]).cuda())
    print(f"[p10 checked accessor] {bad} out-of-range access(es) recorded, first by thread {who} at index {idx}; "
          "no fault raised")
    return ok and bad == 1 and idx == 9


def p11(f):
    a = torch.arange(8.0)
    return _check("p11 pooling", P.pool3(cu(a)), P.oracle_pool3(a))


def p12(f):
    a, b = torch.arange(8.0), torch.arange(8.0)
    return _check("p12 dot_product", P.dot(cu(a), cu(b)), (a * b).sum().reshape(1))


def p13(f):
    if f == "block-boundary":
        a, k = torch.arange(15.0), torch.arange(4.0)
    else:
        a, k = torch.arange(6.0), torch.arange(3.0)
    return _check(f"p13 conv_1d ({f or 'simple'})", P.conv1d(cu(a), cu(k), block=8), P.oracle_conv1d(a, k))


def p14(f):
    a = torch.arange(15.0 if f == "complete" else 8.0)
    return _check(f"p14 prefix_sum ({f or 'simple'})", P.prefix_sum(cu(a), block=8), torch.cumsum(a, 0))


def p15(f):
    a = torch.arange(24.0).view(4, 6)
    return _check("p15 axis_sum", P.axis_sum(cu(a)), a.sum(1))


def p16(f):
    variant = {"single-block": "single_block", "tiled": "tiled"}.get(f, "naive")
    n = 2 if variant == "single_block" else 9 if variant == "tiled" else 2
    a = torch.arange(float(n * n)).view(n, n)
    b = torch.arange(float(n * n)).view(n, n) * 2
    return _check(f"p16 matmul ({variant})", P.matmul(cu(a), cu(b), variant), a @ b, 1e-3)


def p17(f):
    import zero_to_hero_b200.ops.custom_ops  # noqa: F401
    a, k = torch.arange(15.0), torch.arange(4.0)
    return _check("p17 conv1d custom op", torch.ops.z2h.conv1d(cu(a), cu(k)), P.oracle_conv1d(a, k))


def p18(f):
    import zero_to_hero_b200.ops.custom_ops  # noqa: F401
    x = torch.randn(128, generator=torch.Generator().manual_seed(0))
    ok = _check("p18 softmax (gpu)", torch.ops.z2h.softmax(cu(x)), torch.softmax(x, 0), 1e-6)
    return ok and _check("p18 softmax (cpu)", torch.ops.z2h.softmax(x), torch.softmax(x, 0), 1e-6)


def p19(f):
    import zero_to_hero_b200.ops.custom_ops  # noqa: F401
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(16, generator=g), torch.randn(16, 16, generator=g), torch.randn(16, 16, generator=g)
    return _check("p19 attention", torch.ops.z2h.attention(cu(q), cu(k), cu(v)), torch.softmax(k @ q, 0) @ v, 1e-5)


def p20(f):
    import zero_to_hero_b200.ops.custom_ops  # noqa: F401
    a, k = torch.arange(15.0), torch.arange(4.0)
    fn = torch.compile(lambda x, w: torch.ops.z2h.conv1d(x, w)) if f == "compile" else torch.ops.z2h.conv1d
    return _check("p20 conv1d from PyTorch", fn(cu(a), cu(k)), P.oracle_conv1d(a, k))


def p21(f):
    g = torch.Generator().manual_seed(0)
    w = torch.randn(10000, 512, generator=g)
    idx = torch.randint(0, 10000, (8, 512), generator=g)
    ok = True
    for variant in ("coalesced", "2d"):
        ok &= _check(f"p21 embedding ({variant})", P.embedding(idx.cuda(), cu(w), variant), w[idx])
    return ok


def p22(f):
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(42)
    B, S, H, O = 4, 4, 8, 16
    x, gamma, beta = torch.randn(B, S, H, generator=g), torch.rand(H, generator=g) + 0.5, torch.randn(H, generator=g)
    w, bias = torch.randn(O, H, generator=g), torch.randn(O, generator=g)
    ref = F.linear(F.layer_norm(x, (H,), gamma, beta), w, bias)
    if f == "backward":
        xs = [t.clone().requires_grad_(True) for t in (x, gamma, beta, w, bias)]
        dy = torch.randn(B, S, O, generator=g)
        F.linear(F.layer_norm(xs[0], (H,), xs[1], xs[2]), xs[3], xs[4]).backward(dy)
        got = P.ln_linear_bwd(cu(dy), cu(x), cu(gamma), cu(beta), cu(w))
        return all(_check(f"p22 backward {n}", a, r.grad, 1e-4)
                   for n, a, r in zip(["dx", "dgamma", "dbeta", "dw", "dbias"], got, xs))
    fused = f != "unfused"
    return _check(f"p22 layernorm_linear ({'fused' if fused else 'unfused'})",
                  P.ln_linear_fwd(cu(x), cu(gamma), cu(beta), cu(w), cu(bias), fused=fused), ref, 1e-4)


def p23(f):
    a, b = torch.arange(1024.0), torch.arange(1024.0) * 2
    variant = {"tiled": "tiled", "manual-vectorized": "vectorized", "vectorized": "vectorized"}.get(f, "scalar")
    return _check(f"p23 elementwise_add ({variant})", P.elementwise_add(cu(a), cu(b), variant), a + b)


def p24(f):
    a, b = torch.arange(32.0), torch.arange(32.0)
    return _check("p24 warp dot_product", P.warp_dot(cu(a), cu(b)), (a * b).sum().reshape(1), 1e-3)


def _warp(op, n=32):
    v = torch.arange(float(n)) * 0.5 + 1
    return _check(f"{op}", P.warp_op(cu(v), op), P.oracle_warp_op(v, op))


def p25(f):
    ops = ["neighbor_difference", "moving_average_3", "broadcast_shuffle_coordination", "basic_broadcast",
           "conditional_broadcast"]
    sel = [o for o in ops if f and f.replace("-", "_") in o] or ops
    return all(_warp(o, 64 if o == "moving_average_3" else 32) for o in sel)


def p26(f):
    ok = all(_warp(o, 64 if o == "butterfly_conditional_max" else 32)
             for o in ["butterfly_pair_swap", "butterfly_parallel_max", "butterfly_conditional_max",
                       "warp_inclusive_prefix_sum"])
    v = torch.tensor([3., 7., 1., 8., 2., 9., 4., 6.])
    return ok and _check("warp_partition", P.warp_partition(cu(v), 5.0), [3., 1., 2., 4., 7., 8., 9., 6.])


def p27(f):
    a = (torch.arange(128.0) % 80) / 100.0
    ok = _check("p27 block.sum dot", P.block_dot(cu(a), cu(a)), (a * a).sum().reshape(1), 1e-3)
    vals, n = P.block_histogram_bin_extract(cu(a), 0, 8)
    ok &= _check("p27 histogram bin 0", vals, a[(a * 8).floor() == 0])
    return ok and _check("p27 normalize", P.block_normalize(cu(a)), a / a.mean(), 1e-5)


def p28(f):
    a = torch.arange(16384.0) % 10
    w = torch.tensor([1., 2., 3., 2., 1.]) / 9
    return _check("p28 async copy conv", P.async_copy_conv(cu(a), cu(w), bulk=(f == "bulk"))[:1024],
                  P.oracle_async_copy_conv(a[:1024], w), 1e-4)


def p29(f):
    a = torch.arange(1024.0) % 10
    if f == "double-buffer":
        return _check("p29 double_buffered_stencil", P.double_buffer_stencil(cu(a), 3),
                      P.oracle_double_buffer_stencil(a, 3), 1e-4)
    return _check("p29 multi_stage pipeline", P.pipeline_blur(cu(a)), P.oracle_pipeline_blur(a), 1e-4)


def p30(f):
    a, b = torch.arange(16384.0), torch.ones(16384)
    return all(_check(f"p30 {m}", P.access_pattern_add(cu(a), cu(b), m), a + b) for m in ("coalesced", "strided", "reversed"))


def p31(f):
    x, y = torch.arange(4096.0), torch.ones(4096)
    return all(_check(f"p31 saxpy smem={s}", P.occupancy_saxpy(cu(y), cu(x), 2.0, s), 2 * x + y)
               for s in (4096, 16384, 49152))


def p32(f):
    a = torch.arange(8192.0)
    return all(_check(f"p32 stride {s}", P.bank_conflict(cu(a), s), (a + 10) * 2) for s in (1, 2))


def p33(f):
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(1024, 1024, generator=g) * 0.1, torch.randn(1024, 1024, generator=g) * 0.1
    variant = {"tensor-core": "tf32_mma", "tcgen05": "tcgen05"}.get(f, "tiled")
    return _check(f"p33 matmul ({variant})", P.matmul(cu(a), cu(b), variant), a @ b, 2e-2 if variant != "tiled" else 1e-3)


def p34(f):
    a = torch.arange(1024.0) % 7
    if f == "reduction":
        return all(_check(f"p34 cluster reduce dsmem={d}", P.cluster_reduce(cu(a), 256, 4, d), a.sum().reshape(1), 1e-3)
                   for d in (False, True))
    ref = torch.stack([(a[i * 256:(i + 1) * 256] * (i + 1)).sum() for i in range(4)])
    return _check(f"p34 cluster ({f or 'coordination'})", P.cluster_block_sums(cu(a), 256, 4, f == "advanced"), ref, 1e-3)


# ------------------------------------------------------------------------------ benchmarks
def _bench_line(puzzle, variant, n, bytes_moved, fn):
    import json

    from .utils.kernel_bench import peaks, time_kernel
    ms = time_kernel(fn, iters=20, warmup=3, flush=True)
    hbm, _, tag = peaks()
    gbs = bytes_moved / ms / 1e6
    print(json.dumps({"puzzle": puzzle, "variant": variant, "n": n, "us": round(ms * 1e3, 2),
                      "gbs": round(gbs, 1), "frac_hbm": f"{gbs / hbm:.3f} {tag}"}), flush=True)


def bench_p23():
    """Vector add, three kernels, 16 ... 1 Mi elements (and 64 Mi, where DRAM decides)."""
    for n in [16, 128, 1024, 8192, 65536, 1 << 20, 64 << 20]:
        a, b = torch.rand(n, device="cuda"), torch.rand(n, device="cuda")
        for variant in ("scalar", "tiled", "vectorized"):
            _bench_line("p23", variant, n, 12 * n, lambda: P.elementwise_add(a, b, variant))


def bench_p24():
    """One dot product per 32 elements: the warp-shuffle kernel against the library expression,
    1 ... 65536 warps of data."""
    for warps in [1, 16, 256, 4096, 65536, 1 << 20]:
        n = warps * 32
        a, b = torch.rand(n, device="cuda"), torch.rand(n, device="cuda")
        _bench_line("p24", "warp_shuffle", n, 8 * n + 4 * warps, lambda: P.warp_dot(a, b))
        _bench_line("p24", "torch (mul, view, sum)", n, 8 * n + 4 * warps, lambda: (a * b).view(-1, 32).sum(1))


def bench_p30():
    """Coalesced, stride-512 and reversed access over 16 Mi elements."""
    n = 16 << 20
    a, b = torch.rand(n, device="cuda"), torch.rand(n, device="cuda")
    for mode in ("coalesced", "strided", "reversed"):
        _bench_line("p30", mode, n, 12 * n, lambda: P.access_pattern_add(a, b, mode))


def bench_p31():
    """SAXPY over 32 Mi elements with 4, 16 and 48 KiB of shared memory per CTA (occupancy)."""
    n = 32 << 20
    x, y = torch.rand(n, device="cuda"), torch.rand(n, device="cuda")
    for smem in (4096, 16384, 49152):
        _bench_line("p31", f"smem {smem}", n, 12 * n + 4 * n, lambda: P.occupancy_saxpy(y, x, 2.0, smem))


def bench_p32():
    """Shared-memory stride 1 against stride 2 (two-way bank conflict), 8192 and 16 Mi elements."""
    for n in (8192, 16 << 20):
        a = torch.rand(n, device="cuda")
        for stride in (1, 2):
            _bench_line("p32", f"stride {stride}", n, 8 * n, lambda: P.bank_conflict(a, stride))


BENCHMARKS = {"p23": bench_p23, "p24": bench_p24, "p30": bench_p30, "p31": bench_p31, "p32": bench_p32}
PUZZLES = {f"p{i:02d}": globals()[f"p{i:02d}"] for i in range(1, 35)}
FLAGS = ["first-case", "second-case", "third-case", "simple", "block-boundary", "complete", "naive", "single-block",
         "tiled", "compile", "fused", "unfused", "backward", "manual-vectorized", "vectorized", "bulk",
         "multi-stage", "double-buffer", "tensor-core", "tcgen05", "coordination", "reduction", "advanced"]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("puzzle", choices=list(PUZZLES) + ["all"])
    for fl in FLAGS:
        ap.add_argument(f"--{fl}", dest="flag", action="store_const", const=fl)
    ap.add_argument("--benchmark", action="store_true", help="size sweep with timing (p23, p24, p30, p31, p32)")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("the puzzles need a CUDA device", file=sys.stderr)
        return 2
    names = list(PUZZLES) if a.puzzle == "all" else [a.puzzle]
    if a.benchmark:
        todo = [n for n in names if n in BENCHMARKS]
        if not todo:
            print(f"no benchmark for {a.puzzle}; available: {sorted(BENCHMARKS)}", file=sys.stderr)
            return 2
        for n in todo:
            BENCHMARKS[n]()
        return 0
    ok = all(PUZZLES[n](a.flag) for n in names)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
