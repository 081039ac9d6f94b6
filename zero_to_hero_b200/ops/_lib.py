"""ctypes loader for the native libraries built in-tree by `zero_to_hero_b200.build`.

The CUDA library exposes a plain C ABI (raw device pointers + a `cudaStream_t`), so no torch
headers are needed to build it and every call can be captured into a CUDA graph.
On a machine with a GPU a missing library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIBDIR = Path(__file__).resolve().parent.parent / "lib"
_cuda_lib = None
_host_lib = None


class NativeLibraryMissing(RuntimeError):
    pass


def cuda_lib() -> ctypes.CDLL:
    """The sm_100a kernel library (loads it on first use)."""
    global _cuda_lib
    if _cuda_lib is None:
        # Z2H_NATIVE_LIB=bounds selects the self-checking debug build (csrc/common/checked.cuh)
        variant = os.environ.get("Z2H_NATIVE_LIB", "")
        path = _LIBDIR / ("libz2h_bounds.so" if variant == "bounds" else "libz2h.so")
        if not path.exists():
            flag = " --bounds" if variant == "bounds" else ""
            raise NativeLibraryMissing(
                f"{path} is missing: run `python -m zero_to_hero_b200.build{flag}` (needs nvcc)")
        _cuda_lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    return _cuda_lib


def host_lib() -> ctypes.CDLL:
    """The host-only C++ library (micrograd engine, CPU oracles)."""
    global _host_lib
    if _host_lib is None:
        path = _LIBDIR / "libz2h_host.so"
        if not path.exists():
            raise NativeLibraryMissing(
                f"{path} is missing: run `python -m zero_to_hero_b200.build` (needs g++)")
        _host_lib = ctypes.CDLL(str(path))
    return _host_lib


def have_cuda_lib() -> bool:
    return (_LIBDIR / "libz2h.so").exists()


def use_native(t: torch.Tensor) -> bool:
    """True when `t` lives on a GPU, in which case the native kernels must be used."""
    return t.is_cuda


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_status: dict[int, torch.Tensor] = {}


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 status word that bounded device-side waits write to (0 == ok)."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
    return _status[idx]


STATUS_NAMES = {
    0: "ok", 1: "timeout waiting for a TMA stage", 2: "timeout waiting for a free stage",
    3: "timeout waiting for an accumulator", 4: "timeout waiting for accumulator drain",
    5: "timeout waiting for a peer rank", 6: "timeout in an intra-CTA wait", 7: "bad argument",
    8: "out-of-bounds access caught by the checked build",
}
BOUNDS_SITES = {1: "GEMM epilogue row", 2: "GEMM epilogue edge", 3: "GEMM atomic accumulation",
                4: "embedding table row", 5: "embedding output row", 6: "attention forward output",
                7: "attention backward output"}


def describe_status(s: int) -> str:
    if (s & 0xFF) == 8:
        return f"{STATUS_NAMES[8]} (site {s >> 8}: {BOUNDS_SITES.get(s >> 8, '?')})"
    return STATUS_NAMES.get(s, "?")


def check_status(device=None) -> None:
    """Synchronising check of the status word; raises if any kernel gave up on a wait."""
    s = int(status_word(device).item())
    if s != 0:
        status_word(device).zero_()
        raise RuntimeError(f"z2h kernel reported status {s}: {describe_status(s)}")
