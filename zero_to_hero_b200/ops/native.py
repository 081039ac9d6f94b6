"""Raw Python entry points of the sm_100a kernels (one function per C symbol).

Every function takes torch CUDA tensors, launches on the current stream and returns
immediately; nothing here allocates, so all of it can be captured into a CUDA graph. The
autograd-aware, module-level API lives in `zero_to_hero_b200.ops.functional`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_float, c_void_p

import torch

from . import _lib
from ._lib import ptr, stream_ptr

_sigs = {
    "z2h_layernorm_fwd": [c_void_p] * 6 + [c_int, c_int, c_float, c_void_p],
    "z2h_layernorm_bwd_num_partials": [c_int],
    "z2h_layernorm_bwd": [c_void_p] * 10 + [c_int, c_int, c_int, c_void_p],
    "z2h_layernorm_bwd_dxsum": [c_void_p] * 11 + [c_int, c_int, c_int, c_void_p],
    "z2h_embed_fwd": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                      c_void_p, c_void_p],
    "z2h_embed_bwd": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                      c_void_p],
    "z2h_embed_bwd_ordered": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                              c_int, c_void_p],
    "z2h_colsum_bf16_ordered": [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "z2h_flash_bwd_ex": [c_void_p] * 7 + [c_int, c_int, c_int, c_float, c_void_p, ctypes.c_uint,
                         c_void_p, c_int, c_void_p, c_void_p],
    "z2h_ce_fwd_bwd": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_longlong,
                       c_float, c_int, c_int, c_void_p],
    "z2h_reduce_sum": [c_void_p, c_int, c_float, c_void_p, c_int, c_void_p],
    "z2h_gradnorm_partials": [c_void_p, c_longlong, c_void_p, c_void_p],
    "z2h_adamw_step": [c_void_p] * 5 + [c_longlong, c_longlong, c_void_p, c_void_p, c_int,
                                        c_void_p, c_int, c_void_p],
    "z2h_colsum_bf16": [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_void_p],
    "z2h_cast_f32_to_bf16": [c_void_p, c_void_p, c_longlong, c_void_p],
    "z2h_flash_fwd": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "z2h_flash_bwd": [c_void_p] * 7 + [c_int, c_int, c_int, c_void_p, c_void_p],
    "z2h_flash_fwd_dropout": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p,
                              ctypes.c_uint, c_void_p, c_void_p],
    "z2h_flash_bwd_dbias": [c_void_p] * 7 + [c_int, c_int, c_int, c_float, c_void_p, ctypes.c_uint,
                            c_void_p, c_void_p, c_void_p],
    "z2h_flash_bwd_dropout": [c_void_p] * 7 + [c_int, c_int, c_int, c_float, c_void_p, ctypes.c_uint,
                                               c_void_p, c_void_p],
    "z2h_dropout_apply": [c_void_p, c_void_p, c_void_p, c_longlong, c_float, c_void_p, ctypes.c_uint,
                          c_void_p],
}
_fns: dict[str, ctypes._CFuncPtr] = {}


def _f(name: str):
    fn = _fns.get(name)
    if fn is None:
        fn = getattr(_lib.cuda_lib(), name)
        fn.restype = c_int
        fn.argtypes = _sigs[name]
        _fns[name] = fn
    return fn


def _check(rc: int, name: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc} (1 bad argument, 2 tensor map, 3 launch)")


def _is64(t: torch.Tensor) -> int:
    assert t.dtype in (torch.int64, torch.int32)
    return int(t.dtype == torch.int64)


def layernorm_fwd(x, w, b, y, mean, rstd, eps=1e-5):
    M, C = x.numel() // x.shape[-1], x.shape[-1]
    _check(_f("z2h_layernorm_fwd")(ptr(x), ptr(w), ptr(b), ptr(y), ptr(mean), ptr(rstd), M, C,
                                   eps, stream_ptr()), "layernorm_fwd")


def layernorm_bwd_num_partials(M: int) -> int:
    return _f("z2h_layernorm_bwd_num_partials")(M)


def layernorm_bwd(dy, x, w, mean, rstd, dresid, dx, dw, db, scratch, accumulate=True, dxsum=None):
    """`dxsum` (fp32 [C], optional): += column sums of the output dx, i.e. the bias gradient of the
    projection whose output this residual-stream gradient is; scratch then needs 3 * C floats per
    partial row instead of 2 * C."""
    M, C = x.numel() // x.shape[-1], x.shape[-1]
    if dxsum is None:
        assert scratch.numel() >= layernorm_bwd_num_partials(M) * 2 * C
        _check(_f("z2h_layernorm_bwd")(ptr(dy), ptr(x), ptr(w), ptr(mean), ptr(rstd), ptr(dresid),
                                       ptr(dx), ptr(dw), ptr(db), ptr(scratch), M, C, int(accumulate),
                                       stream_ptr()), "layernorm_bwd")
        return
    assert scratch.numel() >= layernorm_bwd_num_partials(M) * 3 * C and dxsum.dtype == torch.float32
    _check(_f("z2h_layernorm_bwd_dxsum")(ptr(dy), ptr(x), ptr(w), ptr(mean), ptr(rstd), ptr(dresid),
                                         ptr(dx), ptr(dw), ptr(db), ptr(dxsum), ptr(scratch), M, C,
                                         int(accumulate), stream_ptr()), "layernorm_bwd_dxsum")


def embed_fwd(idx, wte, wpe, out, T):
    M, C = idx.numel(), wte.shape[1]
    _check(_f("z2h_embed_fwd")(ptr(idx), _is64(idx), ptr(wte), ptr(wpe), ptr(out), M, T, C,
                               wte.shape[0], ptr(_lib.status_word(out.device)), stream_ptr()),
           "embed_fwd")


def embed_bwd(idx, dx, dwte, dwpe, B, T, ordered: bool = False):
    """`ordered`: the token-embedding gradient is summed in ascending position by one writer per
    vocabulary row instead of with atomics (bitwise reproducible, slower)."""
    C = dx.shape[-1]
    _check(_f("z2h_embed_bwd_ordered")(ptr(idx), _is64(idx), ptr(dx), ptr(dwte), ptr(dwpe), B, T, C,
                                       dwte.shape[0], int(ordered), stream_ptr()), "embed_bwd")


def ce_fwd_bwd(logits, targets, losses, v_real, grad_scale, write_grad=True, ignore_index=-100):
    M, Vp = logits.shape
    _check(_f("z2h_ce_fwd_bwd")(ptr(logits), ptr(targets), _is64(targets), ptr(losses), M, v_real,
                                Vp, logits.stride(0), grad_scale, int(write_grad), ignore_index,
                                stream_ptr()), "ce_fwd_bwd")


def reduce_sum(x, out, scale=1.0, accumulate=False):
    _check(_f("z2h_reduce_sum")(ptr(x), x.numel(), scale, ptr(out), int(accumulate), stream_ptr()),
           "reduce_sum")


def gradnorm_partials(g, partials) -> int:
    n = _f("z2h_gradnorm_partials")(ptr(g), g.numel(), ptr(partials), stream_ptr())
    if n < 0:
        raise RuntimeError(f"gradnorm_partials failed with code {n}")
    return n


def adamw_step(p32, g, m, v, p16, n_decay, hyper, partials, num_partials, norm_out, zero_grad=True):
    _check(_f("z2h_adamw_step")(ptr(p32), ptr(g), ptr(m), ptr(v), ptr(p16), p32.numel(), n_decay,
                                ptr(hyper), ptr(partials), num_partials, ptr(norm_out),
                                int(zero_grad), stream_ptr()), "adamw_step")


def colsum_scratch_elems(M: int, N: int) -> int:
    """fp32 elements of scratch the ordered column sum of an M x N matrix uses (up to 128 partial rows)."""
    return min(128, max(1, (M + 127) // 128)) * N


def colsum_bf16(dy, db, accumulate=True, ordered: bool = False, scratch=None):
    """db (+)= column sums of dy. By default up to 128 row slabs are summed by CTAs of their own and
    meet in atomics. `ordered`: bitwise reproducible; with `scratch` (fp32, colsum_scratch_elems) the
    slabs store their partial sums there and a second kernel adds them in slab order, without it one CTA
    sums a whole column block (slow)."""
    M, N = dy.shape
    if scratch is not None:
        assert scratch.dtype == torch.float32 and scratch.numel() >= colsum_scratch_elems(M, N)
    _check(_f("z2h_colsum_bf16_ordered")(ptr(dy), M, N, dy.stride(0), ptr(db), int(accumulate), int(ordered),
                                         ptr(scratch), stream_ptr()), "colsum_bf16")


def cast_f32_to_bf16(src, dst):
    _check(_f("z2h_cast_f32_to_bf16")(ptr(src), ptr(dst), src.numel(), stream_ptr()), "cast")


def flash_fwd(qkv, out, lse, B, T, H, drop_p: float = 0.0, seed=None, site: int = 0):
    """Causal attention forward. With `drop_p` > 0 the attention probabilities are dropped with
    the mask of (`seed` [int64 device tensor of one element], `site`); see ops/dropout.py."""
    if drop_p > 0.0:
        assert seed is not None and seed.dtype == torch.int64 and seed.is_cuda
        _check(_f("z2h_flash_fwd_dropout")(ptr(qkv), ptr(out), ptr(lse), B, T, H, drop_p, ptr(seed), site,
                                           ptr(_lib.status_word(out.device)), stream_ptr()),
               "flash_fwd_dropout")
        return
    _check(_f("z2h_flash_fwd")(ptr(qkv), ptr(out), ptr(lse), B, T, H,
                               ptr(_lib.status_word(out.device)), stream_ptr()), "flash_fwd")


def flash_bwd_stats_elems(B: int, T: int, H: int) -> int:
    """Number of fp32 scratch elements `flash_bwd` needs for its per-row statistics."""
    return 2 * B * H * ((T + 127) // 128 * 128)


def flash_bwd_dq_elems(B: int, T: int, H: int) -> int:
    """Number of fp32 scratch elements `flash_bwd` needs for its dQ accumulation (rows rounded up
    to a multiple of 32: the kernels keep dQ there in a blocked layout)."""
    return (B * T + 31) // 32 * 32 * H * 64


def flash_bwd(qkv, out, dout, lse, dqkv, dq_accum, stats, B, T, H, drop_p: float = 0.0, seed=None,
              site: int = 0, dbias=None, ordered: bool = False):
    """`dbias` (fp32 [3*H*64]): the column sums of `dqkv` as stored are ADDED to it, i.e. the gradient
    of the QKV projection's bias comes out of the attention backward kernels.
    `ordered`: the KV tiles are launched one after the other, so the fp32 accumulation of dQ happens in
    a fixed order (bitwise reproducible, about 1.5x slower; not together with `dbias`)."""
    assert stats.numel() >= flash_bwd_stats_elems(B, T, H)
    assert dq_accum.numel() >= flash_bwd_dq_elems(B, T, H) and dq_accum.dtype == torch.float32
    if ordered:
        assert dbias is None, "the bias by-product is accumulated with atomics"
        if drop_p > 0.0:
            assert seed is not None and seed.dtype == torch.int64 and seed.is_cuda
        _check(_f("z2h_flash_bwd_ex")(ptr(qkv), ptr(out), ptr(dout), ptr(lse), ptr(dqkv), ptr(dq_accum),
                                      ptr(stats), B, T, H, drop_p, ptr(seed) if drop_p > 0.0 else None, site,
                                      None, 1, ptr(_lib.status_word(out.device)), stream_ptr()),
               "flash_bwd_ex")
        return
    if dbias is not None:
        assert dbias.dtype == torch.float32 and dbias.numel() == 3 * H * 64 and dbias.is_contiguous()
        if drop_p > 0.0:
            assert seed is not None and seed.dtype == torch.int64 and seed.is_cuda
        _check(_f("z2h_flash_bwd_dbias")(ptr(qkv), ptr(out), ptr(dout), ptr(lse), ptr(dqkv),
                                         ptr(dq_accum), ptr(stats), B, T, H, drop_p,
                                         ptr(seed) if drop_p > 0.0 else None, site, ptr(dbias),
                                         ptr(_lib.status_word(out.device)), stream_ptr()),
               "flash_bwd_dbias")
        return
    if drop_p > 0.0:
        assert seed is not None and seed.dtype == torch.int64 and seed.is_cuda
        _check(_f("z2h_flash_bwd_dropout")(ptr(qkv), ptr(out), ptr(dout), ptr(lse), ptr(dqkv),
                                           ptr(dq_accum), ptr(stats), B, T, H, drop_p, ptr(seed), site,
                                           ptr(_lib.status_word(out.device)), stream_ptr()),
               "flash_bwd_dropout")
        return
    _check(_f("z2h_flash_bwd")(ptr(qkv), ptr(out), ptr(dout), ptr(lse), ptr(dqkv), ptr(dq_accum),
                               ptr(stats), B, T, H, ptr(_lib.status_word(out.device)),
                               stream_ptr()), "flash_bwd")


def dropout_apply(x, out, drop_p: float, seed, site: int, residual=None):
    """out = dropout(x) (+ residual) over contiguous bf16 tensors; `out` may be `x`. The mask is a
    function of (seed[0], site, element index): applying the call to a gradient with the same seed
    and site is the backward of the forward call (ops/dropout.py restates the mask on the host)."""
    assert x.is_contiguous() and out.is_contiguous() and x.dtype == torch.bfloat16
    assert seed.dtype == torch.int64 and seed.is_cuda
    if residual is not None:
        assert residual.is_contiguous() and residual.numel() == x.numel()
    _check(_f("z2h_dropout_apply")(ptr(x), ptr(residual), ptr(out), x.numel(), drop_p, ptr(seed), site,
                                   stream_ptr()), "dropout_apply")
