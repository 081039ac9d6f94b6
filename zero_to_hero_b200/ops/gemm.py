"""Python entry to the tcgen05 bf16 GEMM family (csrc/gemm/gemm_tcgen05.cu)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

(EPI_NONE, EPI_RESIDUAL, EPI_GELU, EPI_GELU_GRAD, EPI_ATOMIC_ADD, EPI_ACCUMULATE, EPI_GELU_SAVE_GRAD,
 EPI_MUL_AUX, EPI_SLICE_STORE) = range(9)

_configured = False


def _fn():
    global _configured
    lib = _lib.cuda_lib()
    if not _configured:
        lib.z2h_gemm_fold_slices.restype = ctypes.c_int
        lib.z2h_gemm_fold_slices.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p,
                                             ctypes.c_void_p]
        lib.z2h_gemm_bf16_ex.restype = ctypes.c_int
        lib.z2h_gemm_bf16_ex.argtypes = [
            ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong,
            ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong,
            ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
            ctypes.c_int, ctypes.c_int, ctypes.c_int,
            ctypes.c_int, ctypes.c_int,
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong,
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong,
            ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
        ]
        _configured = True
    return lib.z2h_gemm_bf16_ex


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, a_mn: bool = False,
         b_mn: bool = False, epi: int = EPI_NONE, bias: torch.Tensor | None = None,
         residual: torch.Tensor | None = None, aux_out: torch.Tensor | None = None,
         aux_in: torch.Tensor | None = None, split_k: int = 1, max_ctas: int = 0,
         colsum: torch.Tensor | None = None, slice_stride: int = 0) -> torch.Tensor:
    """out[M,N] (op)= A · Bᵀ on the tensor cores.

    `a` is [M,K] (or [K,M] when `a_mn`), `b` is [N,K] (or [K,N] when `b_mn`); both bf16 with a
    unit inner stride. `out` is bf16 or fp32 [M,N]. See csrc/gemm/gemm.h for the epilogues.
    `split_k` > 1 cuts K into that many slices; 0 selects the stream-K schedule (one equal run of
    k-blocks per SM); both need `epi=EPI_ATOMIC_ADD` and an fp32 `out` that already holds the
    value to add to.
    `epi=EPI_SLICE_STORE` with `split_k` = S (fp32 `out`, the first of S slices `slice_stride` elements
    apart): K-slice s of every tile is stored at out + s * slice_stride; `fold_slices` then adds the
    slices to their destination in slice order: split-K without atomics, bitwise reproducible.
    `colsum` (fp32 [N]): the column sums of `out` as stored are ADDED to it by the epilogue, i.e. the
    bias gradient of the layer whose output gradient this GEMM produces comes for free; needs a bf16
    `out`, `split_k == 1` and M, N multiples of 32.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and out.stride(-1) == 1
    M, N = out.shape
    K = a.shape[0] if a_mn else a.shape[1]
    assert (a.shape[1] if a_mn else a.shape[0]) == M, (a.shape, out.shape, a_mn)
    assert (b.shape[1] if b_mn else b.shape[0]) == N, (b.shape, out.shape, b_mn)
    assert (b.shape[0] if b_mn else b.shape[1]) == K
    out_fp32 = out.dtype == torch.float32
    if colsum is not None:
        assert colsum.dtype == torch.float32 and colsum.numel() == N and colsum.is_contiguous()
    aux = aux_out if aux_out is not None else aux_in
    rc = _fn()(
        _lib.ptr(a), int(a_mn), a.stride(0), _lib.ptr(b), int(b_mn), b.stride(0),
        _lib.ptr(out), out.stride(0), int(out_fp32), M, N, K, epi, split_k,
        _lib.ptr(bias), _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
        _lib.ptr(aux_out), _lib.ptr(aux_in), aux.stride(0) if aux is not None else 0,
        _lib.ptr(_lib.status_word(out.device)), max_ctas, _lib.ptr(colsum), int(slice_stride),
        _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"z2h_gemm_bf16 failed with code {rc} for M={M} N={N} K={K}")
    return out


def fold_slices(slices: torch.Tensor, num_slices: int, dst: torch.Tensor) -> None:
    """dst += slices[0] + slices[1] + ... in that order; `slices` holds num_slices * dst.numel() fp32."""
    n = dst.numel()
    assert slices.dtype == torch.float32 and dst.dtype == torch.float32 and dst.is_contiguous()
    assert slices.numel() >= num_slices * n and n % 4 == 0
    _fn()
    rc = _lib.cuda_lib().z2h_gemm_fold_slices(_lib.ptr(slices), num_slices, n, _lib.ptr(dst), _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"z2h_gemm_fold_slices failed with code {rc}")


def set_algo(algo: int) -> None:
    """0: one-CTA kernel (128x256 tiles); 1: CTA-pair kernel (256x256 tiles, cta_group::2) whenever
    M >= 256; 2: automatic choice (default)."""
    _lib.cuda_lib().z2h_gemm_set_algo(int(algo))


def set_fixup(on: bool) -> None:
    """Stream-K with fix-up in the CTA-pair kernel (default off: it measured slower on B200): tile
    counts that leave a ragged last wave are cut into equal runs of k-blocks; a tile shared by two
    runs is finished by one of them."""
    _lib.cuda_lib().z2h_gemm_set_fixup(int(bool(on)))


def get_algo() -> int:
    return int(_lib.cuda_lib().z2h_gemm_get_algo())
