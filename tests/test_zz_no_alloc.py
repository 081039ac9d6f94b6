"""LayerNorm backward through the allocation-free C entry point.

Some users of the native library cannot allocate device memory when they need this op: a C/C++
program that links libz2h.so without PyTorch and has no allocator of its own, or a server that
has already given all device memory to its own pools. `z2h_layernorm_bwd_noalloc` therefore
keeps its scratch in a fixed area inside the library. This test calls it through the exported C
symbol (ctypes), twice in a row on the same inputs, and checks both results against the regular
entry point, which takes a caller-provided scratch buffer. The file name sorts last so that a
run which stops at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(M, C, dev):
    g = torch.Generator(device="cpu").manual_seed(M * 7919 + C)
    x = torch.randn(M, C, generator=g).bfloat16().to(dev)
    w = (torch.randn(C, generator=g) * 0.5 + 1).bfloat16().to(dev)
    dy = torch.randn(M, C, generator=g).bfloat16().to(dev)
    dres = torch.randn(M, C, generator=g).bfloat16().to(dev)
    return x, w, dy, dres


@pytest.mark.parametrize("M,C", [(1000, 768), (4096, 1600), (37, 2048)])
def test_noalloc_entry_point_matches_regular_one_twice(M, C):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.ops import _lib, native as N

    dev = torch.device("cuda")
    lib = _lib.cuda_lib()
    fn = lib.z2h_layernorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 9 + [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    cap = lib.z2h_layernorm_bwd_noalloc_capacity
    cap.restype = ctypes.c_longlong
    assert cap() == 296 * 2 * 2048

    x, w, dy, dres = _inputs(M, C, dev)
    y = torch.empty_like(x)
    mean = torch.empty(M, device=dev)
    rstd = torch.empty(M, device=dev)
    N.layernorm_fwd(x, w, None, y, mean, rstd)

    # the regular entry point, with a scratch buffer the caller allocated
    dx_ref = torch.empty_like(x)
    dw_ref = torch.zeros(C, device=dev)
    db_ref = torch.zeros(C, device=dev)
    scratch = torch.empty(N.layernorm_bwd_num_partials(M) * 2 * C, device=dev)
    N.layernorm_bwd(dy, x, w, mean, rstd, dres, dx_ref, dw_ref, db_ref, scratch, accumulate=False)

    p = _lib.ptr
    for call in range(2):  # the second call finds the first call's leftovers in the scratch area
        dx = torch.full_like(x, float("nan"))
        dw = torch.full((C,), float("nan"), device=dev)
        db = torch.full((C,), float("nan"), device=dev)
        rc = fn(p(dy), p(x), p(w), p(mean), p(rstd), p(dres), p(dx), p(dw), p(db), M, C, 0,
                _lib.stream_ptr())
        assert rc == 0, f"call {call}: z2h_layernorm_bwd_noalloc returned {rc}"
        torch.cuda.synchronize()

        def rel(a, b):
            return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-9)

        assert rel(dx, dx_ref) < 1e-2, (call, rel(dx, dx_ref))
        assert rel(dw, dw_ref) < 1e-4, (call, rel(dw, dw_ref))
        assert rel(db, db_ref) < 1e-4, (call, rel(db, db_ref))


def test_noalloc_entry_point_rejects_oversized_problem():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.ops import _lib

    lib = _lib.cuda_lib()
    fn = lib.z2h_layernorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 9 + [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    # C = 4096 would need twice the built-in scratch: refused before any pointer is touched
    assert fn(None, None, None, None, None, None, None, None, None, 8192, 4096, 0, None) == 4
    # a few wide rows would fit the area, but rows beyond 2048 columns are refused all the same
    assert fn(None, None, None, None, None, None, None, None, None, 8, 4096, 0, None) == 4
    assert fn(None, None, None, None, None, None, None, None, None, 16, 100, 0, None) == 1
