"""Python entry to the teaching primitives (csrc/primitives/*.cu) and their CPU oracles.

Each GPU function takes fp32 CUDA tensors and returns a new tensor; `oracle_*` functions are
plain PyTorch/NumPy restatements on the CPU that the tests and the `puzzles` command line
compare against. The kernels are the CUDA C++ counterparts of the reference's Mojo puzzles
(gpu-mojo/problems/p01 .. p34); the shapes those puzzles hard-code are listed in
`zero_to_hero_b200.puzzles`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import _lib
from ._lib import ptr, stream_ptr

_cache: dict[str, ctypes._CFuncPtr] = {}


def _call(name: str, *args) -> None:
    fn = _cache.get(name)
    if fn is None:
        fn = getattr(_lib.cuda_lib(), name)
        fn.restype = c_int
        _cache[name] = fn
    conv = []
    for a in args:
        if isinstance(a, torch.Tensor) or a is None:
            conv.append(ptr(a))
        elif isinstance(a, float):
            conv.append(c_float(a))
        elif isinstance(a, int):
            conv.append(c_longlong(a) if abs(a) > 2**31 - 1 else c_int(a))
        else:
            conv.append(a)
    rc = fn(*conv)
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc} (1 bad argument, 3 launch failed)")


def _f(t: torch.Tensor) -> torch.Tensor:
    assert t.is_cuda and t.dtype == torch.float32
    return t.contiguous()


def _cdiv(a, b):
    return (a + b - 1) // b


# --------------------------------------------------------------------------- p01 - p08
def add10(a, block=128, vectorized=False):
    a = _f(a)
    out = torch.empty_like(a)
    if vectorized:
        fn = _lib.cuda_lib().z2h_p_add10_vec4
        fn.restype = c_int
        fn.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p]
        rc = fn(ptr(out), ptr(a), a.numel(), stream_ptr())
        if rc:
            raise RuntimeError(f"z2h_p_add10_vec4 failed with code {rc}")
    else:
        _call("z2h_p_add10", out, a, a.numel(), block, stream_ptr())
    return out


def zip_add(a, b, block=128):
    a, b = _f(a), _f(b)
    out = torch.empty_like(a)
    _call("z2h_p_zip_add", out, a, b, a.numel(), block, stream_ptr())
    return out


def add10_2d(a, block=(3, 3)):
    a = _f(a)
    out = torch.empty_like(a)
    _call("z2h_p_add10_2d", out, a, a.shape[0], a.shape[1], block[0], block[1], stream_ptr())
    return out


def broadcast_add(row, col, block=(3, 3)):
    """out[r, c] = row[c] + col[r]."""
    row, col = _f(row).reshape(-1), _f(col).reshape(-1)
    out = torch.empty(col.numel(), row.numel(), device=row.device)
    _call("z2h_p_broadcast_add", out, row, col, col.numel(), row.numel(), block[0], block[1], stream_ptr())
    return out


def add10_shared(a, block=4):
    a = _f(a)
    out = torch.empty_like(a)
    _call("z2h_p_add10_shared", out, a, a.numel(), block, stream_ptr())
    return out


# --------------------------------------------------------------------------- p11 - p15
def pool3(a, block=8):
    a = _f(a)
    out = torch.empty_like(a)
    _call("z2h_p_pool3", out, a, a.numel(), block, stream_ptr())
    return out


def oracle_pool3(a):
    a = a.float().cpu()
    out = a.clone()
    out[1:] += a[:-1]
    out[2:] += a[:-2]
    return out


def dot(a, b, block=8):
    a, b = _f(a), _f(b)
    out = torch.empty(1, device=a.device)
    scratch = torch.empty(_cdiv(a.numel(), 1) + 1, device=a.device)
    _call("z2h_p_dot", out, a, b, a.numel(), block, scratch, stream_ptr())
    return out


def conv1d(a, w, block=8):
    """out[i] = sum_k a[i + k] * w[k], zero beyond the end (correlation with right zero pad)."""
    a, w = _f(a), _f(w)
    out = torch.empty_like(a)
    _call("z2h_p_conv1d", out, a, w, a.numel(), w.numel(), block, stream_ptr())
    return out


def oracle_conv1d(a, w):
    a, w = a.float().cpu(), w.float().cpu()
    n, k = a.numel(), w.numel()
    pad = torch.cat([a, torch.zeros(k - 1)])
    return torch.stack([(pad[i:i + k] * w).sum() for i in range(n)])


def prefix_sum(a, block=8):
    a = _f(a)
    out = torch.empty_like(a)
    scratch = torch.empty(a.numel() + 1, device=a.device)
    _call("z2h_p_prefix_sum", out, a, a.numel(), block, scratch, stream_ptr())
    return out


def axis_sum(a, block=8):
    a = _f(a)
    out = torch.empty(a.shape[0], device=a.device)
    _call("z2h_p_axis_sum", out, a, a.shape[0], a.shape[1], block, stream_ptr())
    return out


# --------------------------------------------------------------------------- p09 / p10
def sliding_window3(a):
    a = _f(a)
    out = torch.empty_like(a)
    _call("z2h_p_sliding_window3", out, a, a.numel(), stream_ptr())
    return out


def oracle_sliding_window3(a):
    a = a.float().cpu()
    out = a.clone()
    out[1:] += a[:-1]
    out[:-1] += a[1:]
    return out


def collaborative_filter(a):
    a = _f(a)
    out = torch.empty_like(a)
    _call("z2h_p_collaborative_filter", out, a, a.numel(), stream_ptr())
    return out


def oracle_collaborative_filter(a):
    a = a.float().cpu()
    out = a.clone()
    n = a.numel()
    if n > 2:
        out[1:n - 1] = a[1:n - 1] + 0.5 * a[0:n - 2]
    return out


def shared_sum_broadcast(a):
    a = _f(a)
    out = torch.empty_like(a)
    _call("z2h_p_shared_sum_broadcast", out, a, a.shape[0], stream_ptr())
    return out


def checked_gather(src, idx):
    """out[t] = src[idx[t]]; returns (out, violations, first_thread, first_index). Bad indices
    read as 0 and are counted instead of faulting."""
    src = _f(src)
    idx = idx.to(torch.int32).contiguous()
    out = torch.empty(idx.numel(), device=src.device)
    status = torch.zeros(3, dtype=torch.int32, device=src.device)
    _call("z2h_p_checked_gather", out, src, idx, idx.numel(), src.numel(), status, stream_ptr())
    st = status.tolist()
    return out, st[0], st[1], st[2]


# --------------------------------------------------------------------------- p16 / p33 matmul
MATMUL_VARIANTS = {"naive": 0, "single_block": 1, "tiled": 2, "tf32_mma": 3}


def matmul(a, b, variant="tiled"):
    """C = A @ B in fp32 storage. "tcgen05" routes through the bf16 tensor-core GEMM of the
    training path (inputs rounded to bf16), the Blackwell twin of the TF32 mma.sync kernel."""
    a, b = _f(a), _f(b)
    M, K = a.shape
    N = b.shape[1]
    if variant == "tcgen05":
        from . import gemm as G
        out = torch.empty(M, N, device=a.device)
        G.gemm(a.bfloat16().contiguous(), b.bfloat16().contiguous(), out, b_mn=True)
        return out
    out = torch.empty(M, N, device=a.device)
    _call("z2h_p_matmul", out, a, b, M, N, K, MATMUL_VARIANTS[variant], stream_ptr())
    return out


def transpose(a):
    a = _f(a)
    out = torch.empty(a.shape[1], a.shape[0], device=a.device)
    _call("z2h_p_transpose", out, a, a.shape[0], a.shape[1], stream_ptr())
    return out


def softmax(a):
    a = _f(a)
    a2 = a.reshape(-1, a.shape[-1])
    out = torch.empty_like(a2)
    _call("z2h_p_softmax", out, a2, a2.shape[0], a2.shape[1], stream_ptr())
    return out.reshape(a.shape)


def attention_vec(q, k, v):
    """softmax(q @ K.T) @ V for one query vector (no scaling, no mask)."""
    q, k, v = _f(q), _f(k), _f(v)
    out = torch.empty(v.shape[1], device=q.device)
    _call("z2h_p_attention_vec", out, q, k, v, k.shape[0], k.shape[1], stream_ptr())
    return out


# --------------------------------------------------------------------------- p21 embedding
def embedding(idx, w, variant="coalesced"):
    idx32 = idx.to(torch.int32).contiguous()
    w = _f(w)
    out = torch.empty(*idx.shape, w.shape[1], device=w.device)
    _call("z2h_p_embedding", out, idx32, w, idx32.numel(), w.shape[1], w.shape[0],
          0 if variant == "coalesced" else 1, stream_ptr())
    return out


# --------------------------------------------------------------------------- p22 LayerNorm + Linear
def ln_linear_fwd(x, gamma, beta, w, bias, eps=1e-5, fused=True):
    x, gamma, beta, w, bias = map(_f, (x, gamma, beta, w, bias))
    H, O = x.shape[-1], w.shape[0]
    x2 = x.reshape(-1, H)
    T = x2.shape[0]
    y = torch.empty(T, O, device=x.device)
    tmp = torch.empty(T * H + H * O, device=x.device)
    _call("z2h_p_ln_linear_fwd", y, x2, gamma, beta, w, bias, T, H, O, float(eps), int(fused), tmp,
          stream_ptr())
    return y.reshape(*x.shape[:-1], O)


def ln_linear_bwd(dy, x, gamma, beta, w, eps=1e-5, deterministic=True):
    """Returns (dx, dgamma, dbeta, dw, dbias)."""
    dy, x, gamma, beta, w = map(_f, (dy, x, gamma, beta, w))
    H, O = x.shape[-1], w.shape[0]
    x2, dy2 = x.reshape(-1, H), dy.reshape(-1, O)
    T = x2.shape[0]
    dx = torch.empty_like(x2)
    dgamma, dbeta = torch.zeros(H, device=x.device), torch.zeros(H, device=x.device)
    dw, dbias = torch.zeros(O, H, device=x.device), torch.zeros(O, device=x.device)
    _call("z2h_p_ln_linear_bwd", dy2, x2, gamma, beta, w, dx, dgamma, dbeta, dw, dbias, T, H, O,
          float(eps), int(deterministic), stream_ptr())
    return dx.reshape(x.shape), dgamma, dbeta, dw, dbias


# --------------------------------------------------------------------------- p23 - p27
def elementwise_add(a, b, variant="vectorized", tile=32):
    a, b = _f(a), _f(b)
    out = torch.empty_like(a)
    v = {"scalar": 0, "tiled": 1, "vectorized": 2}[variant]
    fn = _lib.cuda_lib().z2h_p_ew_add
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p]
    rc = fn(ptr(out), ptr(a), ptr(b), a.numel(), v, tile, stream_ptr())
    if rc:
        raise RuntimeError(f"z2h_p_ew_add failed with code {rc}")
    return out


def warp_dot(a, b):
    """One dot product per group of 32 consecutive elements."""
    a, b = _f(a), _f(b)
    out = torch.zeros(_cdiv(a.numel(), 32), device=a.device)
    _call("z2h_p_warp_dot", out, a, b, a.numel(), stream_ptr())
    return out


def warp_sum_int(a):
    a = a.to(torch.int32).contiguous()
    out = torch.zeros(_cdiv(a.numel(), 32), dtype=torch.int32, device=a.device)
    _call("z2h_p_warp_sum_int", out, a, a.numel(), stream_ptr())
    return out


WARP_OPS = {"neighbor_difference": 0, "moving_average_3": 1, "broadcast_shuffle_coordination": 2,
            "basic_broadcast": 3, "conditional_broadcast": 4, "butterfly_pair_swap": 5,
            "butterfly_parallel_max": 6, "butterfly_conditional_max": 7, "warp_inclusive_prefix_sum": 8}


def warp_op(a, op: str):
    a = _f(a)
    out = torch.empty_like(a)
    _call("z2h_p_warp_op", out, a, a.numel(), WARP_OPS[op], stream_ptr())
    return out


def oracle_warp_op(a, op: str):
    a = a.float().cpu()
    n = a.numel()
    out = torch.empty(n)
    for w0 in range(0, n, 32):
        seg = a[w0:w0 + 32]
        m = seg.numel()
        nxt = lambda k: torch.cat([seg[k:], torch.zeros(min(k, m))])  # noqa: E731 (shuffle_down)
        lane = torch.arange(m)
        if op == "neighbor_difference":
            o = torch.where(lane < 31, nxt(1) - seg, torch.zeros(m))
        elif op == "moving_average_3":
            o = seg.clone()
            for i in range(m):
                gi = w0 + i
                if i < 30:
                    o[i] = (seg[i] + nxt(1)[i] + nxt(2)[i]) / 3
                elif i < 31 and gi < n - 1:
                    o[i] = (seg[i] + nxt(1)[i]) / 2
        elif op == "broadcast_shuffle_coordination":
            scale = (seg[0] + nxt(1)[0] + nxt(2)[0] + nxt(3)[0]) / 4
            o = torch.where(lane < 31, (seg + nxt(1)) * scale, seg * scale)
        elif op == "basic_broadcast":
            o = seg + (seg[0] + nxt(1)[0] + nxt(2)[0] + nxt(3)[0])
        elif op == "conditional_broadcast":
            d = max(float(seg[0]), *(float(nxt(k)[0]) for k in range(1, 8)))
            o = torch.where(seg >= d / 2, seg * 2, seg / 2)
        elif op == "butterfly_pair_swap":
            o = seg.clone()
            for i in range(m):
                o[i] = seg[i ^ 1] if (i ^ 1) < m else 0.0
        elif op == "butterfly_parallel_max":
            o = torch.full((m,), float(seg.max()))
        elif op == "butterfly_conditional_max":
            o = torch.where(lane % 2 == 0, seg.max(), seg.min())
        elif op == "warp_inclusive_prefix_sum":
            o = torch.cumsum(seg, 0)
        else:
            raise KeyError(op)
        out[w0:w0 + m] = o
    return out


def warp_partition(a, pivot: float):
    a = _f(a)
    out = torch.empty_like(a)
    _call("z2h_p_warp_partition", out, a, a.numel(), float(pivot), stream_ptr())
    return out


def block_dot(a, b):
    a, b = _f(a), _f(b)
    out = torch.empty(1, device=a.device)
    _call("z2h_p_block_dot", out, a, b, a.numel(), stream_ptr())
    return out


def block_histogram_bin_extract(a, target_bin: int, num_bins: int = 8):
    """Elements of `a` (values in [0, 1)) that fall into `target_bin`, packed in order."""
    a = _f(a)
    bin_out = torch.zeros_like(a)
    count = torch.zeros(1, dtype=torch.int32, device=a.device)
    _call("z2h_p_block_histogram_bin_extract", a, bin_out, count, a.numel(), target_bin, num_bins,
          stream_ptr())
    n = int(count.item())
    return bin_out[:n], n


def block_normalize(a):
    a = _f(a)
    out = torch.empty_like(a)
    _call("z2h_p_block_normalize", a, out, a.numel(), stream_ptr())
    return out


# --------------------------------------------------------------------------- p28 - p32
def async_copy_conv(a, w5, bulk=False):
    a, w5 = _f(a), _f(w5)
    out = torch.empty_like(a)
    _call("z2h_p_async_copy_conv", out, a, w5, a.numel(), int(bulk), _lib.status_word(a.device),
          stream_ptr())
    return out


def oracle_async_copy_conv(a, w5, tile=256):
    a, w5 = a.float().cpu(), w5.float().cpu()
    out = a.clone()
    n = a.numel()
    for t0 in range(0, n, tile):
        seg = torch.zeros(tile)
        m = min(tile, n - t0)
        seg[:m] = a[t0:t0 + m]
        for l in range(2, tile - 2):
            if t0 + l < n:
                out[t0 + l] = (seg[l - 2:l + 3] * w5).sum()
    return out


def pipeline_blur(a):
    a = _f(a)
    out = torch.empty_like(a)
    _call("z2h_p_pipeline_blur", out, a, a.numel(), stream_ptr())
    return out


def oracle_pipeline_blur(a, tpb=256):
    a = a.float().cpu()
    n = a.numel()
    out = torch.empty(n)
    for b0 in range(0, n, tpb):
        seg = torch.zeros(tpb)
        m = min(tpb, n - b0)
        seg[:m] = a[b0:b0 + m] * 1.1
        blur = torch.empty(tpb)
        for i in range(tpb):
            lo, hi = max(0, i - 2), min(tpb, i + 3)
            blur[i] = seg[lo:hi].sum() / (hi - lo)
        for i in range(m):
            v = blur[i]
            if i > 0:
                v = (v + blur[i - 1]) * 0.6
            if i < tpb - 1:
                v = (v + blur[i + 1]) * 0.6
            out[b0 + i] = v
    return out


def double_buffer_stencil(a, iterations=3):
    a = _f(a)
    out = torch.empty_like(a)
    _call("z2h_p_double_buffer_stencil", out, a, a.numel(), iterations, _lib.status_word(a.device),
          stream_ptr())
    return out


def oracle_double_buffer_stencil(a, iterations=3, tpb=256):
    a = a.float().cpu()
    n = a.numel()
    out = torch.empty(n)
    for b0 in range(0, n, tpb):
        cur = torch.zeros(tpb)
        m = min(tpb, n - b0)
        cur[:m] = a[b0:b0 + m]
        for _ in range(iterations):
            nxt = torch.empty(tpb)
            for i in range(tpb):
                lo, hi = max(0, i - 1), min(tpb, i + 2)
                nxt[i] = cur[lo:hi].sum() / (hi - lo)
            cur = nxt
        out[b0:b0 + m] = cur[:m]
    return out


def access_pattern_add(a, b, mode="coalesced"):
    a, b = _f(a), _f(b)
    if mode == "strided" and a.numel() % 512:
        raise ValueError("the strided pattern needs a length that is a multiple of 512")
    out = torch.empty_like(a)
    _call("z2h_p_access_pattern_add", out, a, b, a.numel(),
          {"coalesced": 0, "strided": 1, "reversed": 2}[mode], stream_ptr())
    return out


def occupancy_saxpy(y, x, alpha: float, smem_bytes: int = 4096):
    y, x = _f(y).clone(), _f(x)
    _call("z2h_p_occupancy_saxpy", y, x, float(alpha), y.numel(), smem_bytes, stream_ptr())
    return y


def bank_conflict(a, stride=1):
    a = _f(a)
    out = torch.empty_like(a)
    _call("z2h_p_bank_conflict", out, a, a.numel(), stride, stream_ptr())
    return out


# --------------------------------------------------------------------------- p34 clusters
def cluster_block_sums(a, block=256, cluster=4, warp_elected=False):
    """One sum per block of in * (block_index + 1), blocks launched in clusters."""
    a = _f(a)
    out = torch.zeros(_cdiv(a.numel(), block), device=a.device)
    _call("z2h_p_cluster_block_sums", out, a, a.numel(), block, cluster, int(warp_elected), stream_ptr())
    return out


def cluster_reduce(a, block=256, cluster=4, dsmem=True):
    """One sum per cluster; with `dsmem` rank 0 reads its peers' shared memory directly."""
    a = _f(a)
    grid = _cdiv(a.numel(), block)
    out = torch.zeros(grid // cluster, device=a.device)
    temp = torch.zeros(grid, device=a.device)
    _call("z2h_p_cluster_reduce", out, a, temp, a.numel(), block, cluster, int(dsmem), stream_ptr())
    return out
