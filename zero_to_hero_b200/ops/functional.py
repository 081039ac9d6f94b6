"""Autograd-aware ops used by the model classes.

On a CUDA device every op runs the hand-written sm_100a kernels (bf16 activations, fp32
statistics / gradients) through `torch.autograd.Function`s; on CPU the same functions fall
back to plain PyTorch in the input dtype, which is also the fp32 oracle the kernel tests
compare against. There is no silent fallback on a GPU: if the native library is missing the
call raises.

Shapes the tensor-core GEMM cannot take (inner sizes that are not multiples of 8 elements,
i.e. 16 bytes for TMA) are routed to `torch.matmul` in bf16 and counted in
`FALLBACK_COUNTS` so tests can assert the hot shapes never take that route.
"""
from __future__ import annotations

import math
from collections import Counter

import torch
import torch.nn.functional as F

from . import _lib, gemm as G, native as N

FALLBACK_COUNTS: Counter = Counter()


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda


_sm_count: dict[int, int] = {}


def sm_count() -> int:
    """SMs of the current CUDA device (148 on a B200; the same figure is assumed without a GPU)."""
    if not torch.cuda.is_available():
        return 148
    d = torch.cuda.current_device()
    if d not in _sm_count:
        _sm_count[d] = torch.cuda.get_device_properties(d).multi_processor_count
    return _sm_count[d]


def pick_split_k(tiles: int, k_blocks: int, num_sms: int | None = None, min_kb: int = 16) -> int:
    """Split-K factor for a weight-gradient GEMM (few output tiles, very long K).

    `tiles` counts 128 x 256 output tiles (one per SM); the kernel that runs them works on CTA
    pairs with 256 x 256 tiles, so the model below uses half as many tiles and half as many
    workers. Cost of a factor s, in k-blocks of main loop: waves(s) * ceil(k_blocks / s) plus
    2 * s for the extra atomic accumulation traffic. Returns 1 (plain deterministic accumulation)
    when the tiles alone fill the machine for several waves.
    """
    if num_sms is None:
        num_sms = sm_count()
    if tiles >= 4 * num_sms or k_blocks < 2 * min_kb:
        return 1
    pair_tiles, workers = max(1, (tiles + 1) // 2), max(1, num_sms // 2)
    best, best_cost = 1, float("inf")
    for s in range(1, 17):
        if s > 1 and k_blocks // s < min_kb:
            break
        cost = math.ceil(pair_tiles * s / workers) * math.ceil(k_blocks / s) + 2 * s
        if cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def _gemm_ok(*dims: int) -> bool:
    return all(d % 8 == 0 for d in dims)


# --------------------------------------------------------------------------------------------
# linear
# --------------------------------------------------------------------------------------------
class _Linear(torch.autograd.Function):
    """y = act(x @ w.T + b) (+ residual) on the tcgen05 GEMM; act in {None, "gelu_tanh"}."""

    @staticmethod
    def forward(ctx, x, w, b, act, residual):
        K = x.shape[-1]
        Nout = w.shape[0]
        x2 = x.reshape(-1, K)
        if x2.dtype != torch.bfloat16:
            x2 = x2.bfloat16()
        x2 = x2.contiguous()
        w16 = w if w.dtype == torch.bfloat16 else w.detach().bfloat16()
        b16 = None if b is None else (b if b.dtype == torch.bfloat16 else b.detach().bfloat16())
        M = x2.shape[0]
        y = torch.empty(M, Nout, device=x.device, dtype=torch.bfloat16)
        pre = None
        if act == "gelu_tanh":
            pre = torch.empty_like(y)
            G.gemm(x2, w16, y, bias=b16, aux_out=pre, epi=G.EPI_GELU)
        elif residual is not None:
            r2 = residual.reshape(M, Nout)
            r2 = (r2 if r2.dtype == torch.bfloat16 else r2.bfloat16()).contiguous()
            G.gemm(x2, w16, y, bias=b16, residual=r2, epi=G.EPI_RESIDUAL)
        else:
            G.gemm(x2, w16, y, bias=b16)
        ctx.save_for_backward(x2, w16, pre)
        ctx.has_bias = b is not None
        ctx.has_res = residual is not None
        ctx.x_shape = x.shape
        ctx.w_dtype = w.dtype
        ctx.b_dtype = None if b is None else b.dtype
        ctx.x_dtype = x.dtype
        ctx.res_dtype = None if residual is None else residual.dtype
        return y.reshape(*x.shape[:-1], Nout)

    @staticmethod
    def backward(ctx, dy):
        x2, w16, pre = ctx.saved_tensors
        M, K = x2.shape
        Nout = w16.shape[0]
        dy2 = dy.reshape(M, Nout)
        dy2 = (dy2 if dy2.dtype == torch.bfloat16 else dy2.bfloat16()).contiguous()
        dres = dy2.reshape(dy.shape).to(ctx.res_dtype) if ctx.has_res else None
        if pre is not None:
            dy2 = _gelu_grad_mul(dy2, pre)  # dpre = dy * gelu'(pre)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx2 = torch.empty(M, K, device=dy.device, dtype=torch.bfloat16)
            G.gemm(dy2, w16, dx2, b_mn=True)
            dx = dx2.reshape(ctx.x_shape).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw32 = torch.zeros(Nout, K, device=dy.device, dtype=torch.float32)
            tiles = math.ceil(Nout / 128) * math.ceil(K / 256)
            sk = pick_split_k(tiles, math.ceil(M / 64))
            G.gemm(dy2, x2, dw32, a_mn=True, b_mn=True, epi=G.EPI_ATOMIC_ADD, split_k=sk)
            dw = dw32.to(ctx.w_dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db32 = torch.zeros(Nout, device=dy.device, dtype=torch.float32)
            N.colsum_bf16(dy2, db32, accumulate=True)
            db = db32.to(ctx.b_dtype)
        return dx, dw, db, None, dres


def _gelu_grad_mul(dy: torch.Tensor, pre: torch.Tensor) -> torch.Tensor:
    x = pre.float()
    k0, k1 = 0.7978845608028654, 0.044715
    u = k0 * (x + k1 * x * x * x)
    t = torch.tanh(u)
    g = 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * k0 * (1 + 3 * k1 * x * x)
    return (dy.float() * g).bfloat16()


def linear(x, w, b=None, act: str | None = None, residual=None):
    """`act(x @ w.T + b) + residual`; act is None or "gelu_tanh" (not both act and residual)."""
    assert not (act and residual is not None)
    K, Nout = x.shape[-1], w.shape[0]
    if _native(x) and _gemm_ok(K, Nout):
        return _Linear.apply(x, w, b, act, residual)
    if _native(x):
        FALLBACK_COUNTS["linear"] += 1
        y = F.linear(x.bfloat16(), w.bfloat16(), None if b is None else b.bfloat16())
    else:
        y = F.linear(x, w, b)
    if act == "gelu_tanh":
        y = F.gelu(y, approximate="tanh")
    if residual is not None:
        y = y + residual
    return y


# --------------------------------------------------------------------------------------------
# layer norm
# --------------------------------------------------------------------------------------------
class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        x2 = (x2 if x2.dtype == torch.bfloat16 else x2.bfloat16()).contiguous()
        w16 = w if w.dtype == torch.bfloat16 else w.detach().bfloat16()
        b16 = None if b is None else (b if b.dtype == torch.bfloat16 else b.detach().bfloat16())
        M = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(M, device=x.device, dtype=torch.float32)
        rstd = torch.empty_like(mean)
        N.layernorm_fwd(x2, w16, b16, y, mean, rstd, eps)
        ctx.save_for_backward(x2, w16, mean, rstd)
        ctx.meta = (x.shape, x.dtype, w.dtype, None if b is None else b.dtype)
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w16, mean, rstd = ctx.saved_tensors
        shape, x_dtype, w_dtype, b_dtype = ctx.meta
        M, C = x2.shape
        dy2 = dy.reshape(M, C)
        dy2 = (dy2 if dy2.dtype == torch.bfloat16 else dy2.bfloat16()).contiguous()
        dx = torch.empty_like(x2)
        dw = torch.empty(C, device=dy.device, dtype=torch.float32)
        db = torch.empty_like(dw) if b_dtype is not None else None
        scratch = torch.empty(N.layernorm_bwd_num_partials(M) * 2 * C, device=dy.device,
                              dtype=torch.float32)
        N.layernorm_bwd(dy2, x2, w16, mean, rstd, None, dx, dw, db, scratch, accumulate=False)
        return (dx.reshape(shape).to(x_dtype), dw.to(w_dtype),
                None if db is None else db.to(b_dtype), None)


def layer_norm(x, w, b=None, eps: float = 1e-5):
    C = x.shape[-1]
    if _native(x) and C % 8 == 0 and C <= 2048:
        return _LayerNorm.apply(x, w, b, eps)
    if _native(x):
        FALLBACK_COUNTS["layer_norm"] += 1
    return F.layer_norm(x, (C,), w, b, eps)


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------
class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, num_heads):
        B, T, C3 = qkv.shape
        C = C3 // 3
        q2 = qkv.reshape(B * T, C3)
        q2 = (q2 if q2.dtype == torch.bfloat16 else q2.bfloat16()).contiguous()
        out = torch.empty(B * T, C, device=qkv.device, dtype=torch.bfloat16)
        lse = torch.empty(B, num_heads, T, device=qkv.device, dtype=torch.float32)
        N.flash_fwd(q2, out, lse, B, T, num_heads)
        ctx.save_for_backward(q2, out, lse)
        ctx.meta = (B, T, num_heads, qkv.dtype)
        return out.reshape(B, T, C)

    @staticmethod
    def backward(ctx, dout):
        q2, out, lse = ctx.saved_tensors
        B, T, H, dtype = ctx.meta
        C = H * 64
        d2 = dout.reshape(B * T, C)
        d2 = (d2 if d2.dtype == torch.bfloat16 else d2.bfloat16()).contiguous()
        dqkv = torch.empty_like(q2)
        dq_accum = torch.empty(N.flash_bwd_dq_elems(B, T, H), device=dout.device, dtype=torch.float32)
        stats = torch.empty(N.flash_bwd_stats_elems(B, T, H), device=dout.device, dtype=torch.float32)
        N.flash_bwd(q2, out, d2, lse, dqkv, dq_accum, stats, B, T, H)
        return dqkv.reshape(B, T, 3 * C).to(dtype), None


def causal_attention(qkv: torch.Tensor, num_heads: int, dropout_p: float = 0.0) -> torch.Tensor:
    """Causal multi-head self-attention over a packed [B, T, 3C] projection; returns [B, T, C]."""
    B, T, C3 = qkv.shape
    C = C3 // 3
    hd = C // num_heads
    if _native(qkv) and hd == 64 and dropout_p == 0.0:
        return _FlashAttention.apply(qkv, num_heads)
    if _native(qkv):
        FALLBACK_COUNTS["attention"] += 1
    q, k, v = qkv.split(C, dim=-1)
    q = q.view(B, T, num_heads, hd).transpose(1, 2)
    k = k.view(B, T, num_heads, hd).transpose(1, 2)
    v = v.view(B, T, num_heads, hd).transpose(1, 2)
    y = F.scaled_dot_product_attention(q, k, v, is_causal=True, dropout_p=dropout_p)
    return y.transpose(1, 2).contiguous().view(B, T, C)


# --------------------------------------------------------------------------------------------
# embedding
# --------------------------------------------------------------------------------------------
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, wte, wpe):
        B, T = idx.shape
        C = wte.shape[1]
        wte16 = wte if wte.dtype == torch.bfloat16 else wte.detach().bfloat16()
        wpe16 = None if wpe is None else (wpe if wpe.dtype == torch.bfloat16 else wpe.detach().bfloat16())
        out = torch.empty(B * T, C, device=idx.device, dtype=torch.bfloat16)
        idxc = idx.contiguous()
        N.embed_fwd(idxc, wte16, wpe16, out, T)
        ctx.save_for_backward(idxc)
        ctx.meta = (B, T, wte.shape, wte.dtype, None if wpe is None else (wpe.shape, wpe.dtype))
        return out.reshape(B, T, C)

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        B, T, wshape, wdtype, pmeta = ctx.meta
        C = wshape[1]
        d2 = dout.reshape(B * T, C)
        d2 = (d2 if d2.dtype == torch.bfloat16 else d2.bfloat16()).contiguous()
        dwte = torch.zeros(wshape, device=dout.device, dtype=torch.float32)
        dwpe = None
        if pmeta is not None:
            dwpe = torch.zeros(pmeta[0], device=dout.device, dtype=torch.float32)
        N.embed_bwd(idx, d2, dwte, dwpe, B, T)
        return None, dwte.to(wdtype), None if dwpe is None else dwpe.to(pmeta[1])


def embedding(idx: torch.Tensor, wte: torch.Tensor, wpe: torch.Tensor | None = None) -> torch.Tensor:
    """wte[idx] + wpe[arange(T)] (the position table may be longer than T)."""
    B, T = idx.shape
    if _native(idx) and wte.shape[1] % 8 == 0:
        return _Embedding.apply(idx, wte, wpe)
    out = F.embedding(idx, wte)
    if wpe is not None:
        out = out + wpe[:T]
    return out


# --------------------------------------------------------------------------------------------
# cross entropy
# --------------------------------------------------------------------------------------------
class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, v_real):
        M, V = logits.shape
        buf = logits.detach().bfloat16().clone() if logits.dtype == torch.bfloat16 else logits.detach().bfloat16()
        if buf.stride(0) % 8 != 0:
            raise ValueError("logits row pitch must be a multiple of 8 elements")
        losses = torch.empty(M, device=logits.device, dtype=torch.float32)
        N.ce_fwd_bwd(buf, targets.contiguous(), losses, v_real, 1.0 / M, write_grad=True)
        ctx.save_for_backward(buf)
        ctx.dtype = logits.dtype
        return losses.mean()

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return (dlogits.float() * g).to(ctx.dtype), None, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, v_real: int | None = None) -> torch.Tensor:
    """Mean softmax cross-entropy over rows; columns >= v_real are vocabulary padding."""
    V = logits.shape[-1]
    v_real = V if v_real is None else v_real
    if _native(logits) and V % 8 == 0:
        return _CrossEntropy.apply(logits.reshape(-1, V), targets.reshape(-1), v_real)
    if _native(logits):
        FALLBACK_COUNTS["cross_entropy"] += 1
    return F.cross_entropy(logits.reshape(-1, V)[:, :v_real].float(), targets.reshape(-1))
