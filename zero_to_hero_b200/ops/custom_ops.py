"""PyTorch custom operators over the teaching kernels.

The reference registers its Mojo kernels as framework ops (`@compiler.register` structs with a
GPU and a CPU target, gpu-mojo/problems/p17..p22/op/*.mojo) and calls them from MAX graphs,
`CustomOpLibrary` and a `torch.autograd.Function` (p17.py:48-64, p20.py:20-37, p22.py:62-112).
Here the same five ops are `torch.library.custom_op`s in the `z2h` namespace:

    torch.ops.z2h.conv1d(input, kernel)                     p17 / p20
    torch.ops.z2h.softmax(input)                            p18
    torch.ops.z2h.attention(q, k, v)                        p19
    torch.ops.z2h.embedding(indices, weights)               p21
    torch.ops.z2h.layernorm_linear(x, gamma, beta, w, b)    p22 (differentiable)

Each op has a CUDA kernel (csrc/primitives) and a CPU kernel in plain PyTorch that doubles as the
oracle, a fake (meta) kernel so the op traces under torch.compile / export, and
`layernorm_linear` has a registered backward that calls the fused backward kernel.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import primitives as P


# ------------------------------------------------------------------------------ conv1d
@torch.library.custom_op("z2h::conv1d", mutates_args=(), device_types="cuda")
def conv1d(input: torch.Tensor, kernel: torch.Tensor) -> torch.Tensor:
    return P.conv1d(input, kernel, block=128)


@conv1d.register_kernel("cpu")
def _(input, kernel):
    k = kernel.numel()
    padded = torch.cat([input, input.new_zeros(k - 1)])
    return padded.unfold(0, k, 1) @ kernel


@conv1d.register_fake
def _(input, kernel):
    return torch.empty_like(input)


# ------------------------------------------------------------------------------ softmax
@torch.library.custom_op("z2h::softmax", mutates_args=(), device_types="cuda")
def softmax(input: torch.Tensor) -> torch.Tensor:
    return P.softmax(input)


@softmax.register_kernel("cpu")
def _(input):
    e = torch.exp(input - input.max(dim=-1, keepdim=True).values)
    return e / e.sum(dim=-1, keepdim=True)


@softmax.register_fake
def _(input):
    return torch.empty_like(input)


# ------------------------------------------------------------------------------ attention
@torch.library.custom_op("z2h::attention", mutates_args=(), device_types="cuda")
def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    return P.attention_vec(q, k, v)


@attention.register_kernel("cpu")
def _(q, k, v):
    return torch.softmax(k @ q, dim=0) @ v


@attention.register_fake
def _(q, k, v):
    return q.new_empty(v.shape[1])


# ------------------------------------------------------------------------------ embedding
@torch.library.custom_op("z2h::embedding", mutates_args=(), device_types="cuda")
def embedding(indices: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    return P.embedding(indices, weights, "coalesced")


@embedding.register_kernel("cpu")
def _(indices, weights):
    ok = (indices >= 0) & (indices < weights.shape[0])
    return weights[indices.clamp(0, weights.shape[0] - 1)] * ok.unsqueeze(-1)


@embedding.register_fake
def _(indices, weights):
    return weights.new_empty(*indices.shape, weights.shape[1])


# ------------------------------------------------------------------------------ layernorm + linear
@torch.library.custom_op("z2h::layernorm_linear", mutates_args=(), device_types="cuda")
def layernorm_linear(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, weight: torch.Tensor,
                     bias: torch.Tensor) -> torch.Tensor:
    return P.ln_linear_fwd(x, gamma, beta, weight, bias, fused=True)


@layernorm_linear.register_kernel("cpu")
def _(x, gamma, beta, weight, bias):
    return F.linear(F.layer_norm(x, (x.shape[-1],), gamma, beta, 1e-5), weight, bias)


@layernorm_linear.register_fake
def _(x, gamma, beta, weight, bias):
    return x.new_empty(*x.shape[:-1], weight.shape[0])


@torch.library.custom_op("z2h::layernorm_linear_backward", mutates_args=(), device_types="cuda")
def layernorm_linear_backward(grad: torch.Tensor, x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor,
                              weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor,
                                                             torch.Tensor, torch.Tensor]:
    return P.ln_linear_bwd(grad, x, gamma, beta, weight, deterministic=True)


@layernorm_linear_backward.register_kernel("cpu")
def _(grad, x, gamma, beta, weight):
    # closed form (custom-op kernels run below autograd, so it cannot be asked for these)
    H = x.shape[-1]
    mean = x.mean(-1, keepdim=True)
    inv = torch.rsqrt(x.var(-1, unbiased=False, keepdim=True) + 1e-5)
    xh = (x - mean) * inv
    ln = xh * gamma + beta
    g2, ln2 = grad.reshape(-1, grad.shape[-1]), ln.reshape(-1, H)
    dln = grad @ weight
    gg = dln * gamma
    dx = inv * (gg - gg.mean(-1, keepdim=True) - xh * (gg * xh).mean(-1, keepdim=True))
    return (dx, (dln * xh).reshape(-1, H).sum(0), dln.reshape(-1, H).sum(0), g2.t() @ ln2, g2.sum(0))


@layernorm_linear_backward.register_fake
def _(grad, x, gamma, beta, weight):
    return (torch.empty_like(x), torch.empty_like(gamma), torch.empty_like(beta), torch.empty_like(weight),
            weight.new_empty(weight.shape[0]))


def _ln_linear_setup(ctx, inputs, output):
    x, gamma, beta, weight, _ = inputs
    ctx.save_for_backward(x, gamma, beta, weight)


def _ln_linear_backward(ctx, grad):
    x, gamma, beta, weight = ctx.saved_tensors
    dx, dgamma, dbeta, dw, dbias = torch.ops.z2h.layernorm_linear_backward(grad.contiguous(), x, gamma, beta, weight)
    return dx, dgamma, dbeta, dw, dbias


layernorm_linear.register_autograd(_ln_linear_backward, setup_context=_ln_linear_setup)
