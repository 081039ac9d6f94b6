"""Per-role clock timelines of the tensor-core kernels (`csrc/common/trace.cuh`).

The GEMM and attention kernels carry `Z2H_TRACE()` marks that compile to nothing in the product build.
This tool builds the named kernel's sources once more with `-DZ2H_KERNEL_TRACE` into
`build/trace/`, runs one launch on the shape of the GPT-2 124M step and prints, for a few CTAs, when
each role (copy warp, MMA-issuing thread, one epilogue / compute warp) passed its marks, in SM cycles:

    python -m zero_to_hero_b200.utils.kernel_trace gemm --N 3072 --K 768 --epi mul_aux
    python -m zero_to_hero_b200.utils.kernel_trace flash_bwd
    python -m zero_to_hero_b200.utils.kernel_trace flash_fwd

This is how the numbers quoted in the kernels' comments were obtained (a tile's main loop against its
epilogue in the GEMM, the MMA thread's issue times and the compute warps' phases in the attention
backward). A traced launch runs a few per cent slower than the product kernel.
"""
from __future__ import annotations

import argparse
import ctypes
import subprocess
from pathlib import Path

import numpy as np
import torch

from .. import build as _build

TRACE_DIR = _build.ROOT / "build" / "trace"
SOURCES = {
    "gemm": ["gemm/gemm_tcgen05.cu", "gemm/gemm_tcgen05_2cta.cu", "common/tma_desc.cu"],
    "flash_bwd": ["attn/flash_bwd.cu", "common/tma_desc.cu"],
    "flash_fwd": ["attn/flash_fwd.cu", "common/tma_desc.cu"],
}
EPI = {"bias": 0, "residual": 1, "gelu": 2, "gelu_grad": 3, "gelu_save_grad": 6, "mul_aux": 7}


def build_trace_lib(name: str) -> ctypes.CDLL:
    """The library of one kernel family with the marks compiled in, cached under build/trace/ by the
    content of its sources and of every header."""
    import hashlib
    srcs = [_build.CSRC / s for s in SOURCES[name]]
    h = hashlib.sha1()
    for p in sorted(srcs + [q for q in _build.CSRC.rglob("*") if q.suffix in (".cuh", ".h")]):
        h.update(p.read_bytes())
    lib = TRACE_DIR / f"libz2h_trace_{name}.{h.hexdigest()[:12]}.so"
    if not lib.exists():
        TRACE_DIR.mkdir(parents=True, exist_ok=True)
        for old in TRACE_DIR.glob(f"libz2h_trace_{name}.*.so"):
            old.unlink()
        cmd = [_build._nvcc(), *_build.NVCC_FLAGS, "-DZ2H_KERNEL_TRACE=1", "-I", str(_build.CSRC), "-shared", "-o",
               str(lib), *map(str, srcs), "-lcuda"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"trace build failed: {r.stderr[-2000:]}")
    return ctypes.CDLL(str(lib))


def _read(lib, fn: str) -> np.ndarray:
    buf = np.zeros((4, 3, 512), dtype=np.int64)  # [traced CTA][role][mark]
    f = getattr(lib, fn)
    f.restype = ctypes.c_int
    if f(buf.ctypes.data_as(ctypes.c_void_p)) != 0:
        raise RuntimeError(f"{fn} failed")
    return buf


def _marks(row: np.ndarray, t0: int) -> list[int]:
    row = row[row > 0]
    return [int(x - t0) for x in row]


def trace_gemm(a) -> None:
    lib = build_trace_lib("gemm")
    f = lib.z2h_gemm_bf16
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong,
                  ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                  ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong,
                  ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    M, N, K, dev = a.M, a.N, a.K, "cuda"
    A = torch.randn(M, K, device=dev).bfloat16()
    B = torch.randn(N, K, device=dev).bfloat16()
    C = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
    other = torch.randn(M, N, device=dev).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    epi = EPI[a.epi]
    has_bias = a.epi in ("bias", "residual", "gelu", "gelu_save_grad")

    def run():
        rc = f(A.data_ptr(), 0, K, B.data_ptr(), 0, K, C.data_ptr(), N, 0, M, N, K, epi, 1,
               bias.data_ptr() if has_bias else None, other.data_ptr() if a.epi == "residual" else None, N,
               other.data_ptr() if a.epi in ("gelu", "gelu_save_grad") else None,
               other.data_ptr() if a.epi in ("gelu_grad", "mul_aux") else None, N, status.data_ptr(), 0, None)
        if rc != 0:
            raise RuntimeError(f"gemm returned {rc}")

    for _ in range(3):
        flush.zero_()
        run()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flush.zero_()
    s.record()
    run()
    e.record()
    torch.cuda.synchronize()
    buf = _read(lib, "z2h_gemm_trace_read_pair")
    mma = buf[0][1][buf[0][1] > 0]
    if len(mma) == 0:
        print("no marks from the CTA-pair kernel (the shape took the one-CTA kernel)")
        return
    t0 = int(mma[0])
    ep = _marks(buf[0][2], t0)
    print(f"gemm M{M} N{N} K{K} epi={a.epi}: {s.elapsed_time(e) * 1000:.1f} us, status {int(status.item())}")
    print("epilogue warp 2 of CTA 0, per tile: accumulator ready at / epilogue cycles / then waited for the next one")
    for i in range(0, len(ep) - 1, 2):
        waited = ep[i + 2] - ep[i + 1] if i + 2 < len(ep) else -1
        print(f"  tile {i // 2:2d}: {ep[i]:8d}  {ep[i + 1] - ep[i]:6d}  {waited:6d}")
    gaps = np.diff(mma)
    print("MMA thread, gaps between marks (stage ready -> 4 MMAs issued + commit -> next stage ready ...), first 3 tiles:")
    per_tile = 2 * ((K + 63) // 64)
    for t in range(min(3, len(gaps) // per_tile)):
        print("  ", [int(x) for x in gaps[t * per_tile:(t + 1) * per_tile]])


def trace_flash(a, which: str) -> None:
    lib = build_trace_lib(which)
    B, T, H, dev = a.B, a.T, a.H, "cuda"
    C = H * 64
    torch.manual_seed(0)
    qkv = (torch.randn(B * T, 3 * C, device=dev) * 0.5).bfloat16()
    out = torch.randn(B * T, C, device=dev).bfloat16()
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    if which == "flash_fwd":
        lse = torch.empty(B, H, T, device=dev)
        f = lib.z2h_flash_fwd
        f.restype = ctypes.c_int
        f.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3 + [ctypes.c_void_p, ctypes.c_void_p]

        def run():
            if f(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), B, T, H, status.data_ptr(), None) != 0:
                raise RuntimeError("flash_fwd failed")
        reader = "z2h_flash_fwd_trace_read"
    else:
        dout = torch.randn(B * T, C, device=dev).bfloat16()
        lse = torch.randn(B, H, T, device=dev).abs() + 3
        dqkv = torch.empty_like(qkv)
        dq = torch.empty(((B * T + 31) // 32 * 32) * C, device=dev)
        stats = torch.empty(2 * B * H * ((T + 127) // 128 * 128), device=dev)
        f = lib.z2h_flash_bwd
        f.restype = ctypes.c_int
        f.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 3 + [ctypes.c_void_p, ctypes.c_void_p]

        def run():
            if f(qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(), dqkv.data_ptr(), dq.data_ptr(),
                 stats.data_ptr(), B, T, H, status.data_ptr(), None) != 0:
                raise RuntimeError("flash_bwd failed")
        reader = "z2h_flash_bwd_trace_read"
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    run()
    e.record()
    torch.cuda.synchronize()
    buf = _read(lib, reader)
    mma_row = buf[0][1][buf[0][1] > 0]
    t0 = int(mma_row[0]) if len(mma_row) else 0
    print(f"{which} B{B} T{T} H{H}: {s.elapsed_time(e) * 1000:.1f} us (all launches), status {int(status.item())}")
    if which == "flash_bwd":
        # CTA 0 handles KV tile 0 and therefore every query tile
        prod, mma, cw = _marks(buf[0][0], t0), _marks(buf[0][1], t0), _marks(buf[0][2], t0)
        print("copy warp: K/V issued, then each query tile's stage issued at:", prod)
        print("MMA thread (S^T/dP^T and dV): start, operands ready, first S^T issued:", mma[:3])
        m = mma[3:]
        for it in range(len(m) // 3):
            x = m[3 * it:3 * it + 3]
            print(f"  tile {it}: S^T/dP^T of the next tile issued {x[0]:7d}  P^T/dS^T ready {x[1]:7d}  dV issued {x[2]:7d}")
        c = cw[1:]
        print("first compute warp, per query tile: stage ready / scores ready / scores in registers / "
              "P^T, dS^T written / handed over / dQ of the previous tile added to the fp32 buffer")
        for it in range(len(c) // 6):
            x = c[6 * it:6 * it + 6]
            print(f"  tile {it}: {x[0]:7d} {x[1]:7d} {x[2]:7d} {x[3]:7d} {x[4]:7d} {x[5]:7d}")
    else:
        for role, name in enumerate(("copy warp", "MMA thread", "softmax warp 0")):
            print(f"{name}, cycles since the MMA thread's first mark (first 64 marks):", _marks(buf[0][role], t0)[:64])


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["gemm", "flash_bwd", "flash_fwd"])
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=3072)
    ap.add_argument("--K", type=int, default=768)
    ap.add_argument("--epi", default="bias", choices=sorted(EPI))
    ap.add_argument("--B", type=int, default=16)
    ap.add_argument("--T", type=int, default=1024)
    ap.add_argument("--H", type=int, default=12)
    a = ap.parse_args()
    if a.kernel == "gemm":
        trace_gemm(a)
    else:
        trace_flash(a, a.kernel)


if __name__ == "__main__":
    main()
