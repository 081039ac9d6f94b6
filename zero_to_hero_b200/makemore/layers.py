"""A hand-rolled module system on raw tensors (nn/makemore/2_2_mlp_modularlized.py:8-154 and
4_1_wavenet.py:97-150 of the reference): `Module` with parameter / buffer / sub-module
registries, `Linear` (Kaiming-scaled), `Embedding`, `Flatten`, `FlattenConsecutive`
(hierarchical pair merging), `BatchNorm1d` over all-but-last dimensions with running
statistics, `Tanh`, `Sequential`."""
from __future__ import annotations

import torch


class Module:
    def __init__(self):
        object.__setattr__(self, "_parameters", {})
        object.__setattr__(self, "_buffers", {})
        object.__setattr__(self, "_modules", {})
        object.__setattr__(self, "training", True)

    def __setattr__(self, name, value):
        if isinstance(value, Module):
            self._modules[name] = value
        object.__setattr__(self, name, value)

    def register_parameter(self, name: str, t: torch.Tensor) -> torch.Tensor:
        t.requires_grad_(True)
        self._parameters[name] = t
        object.__setattr__(self, name, t)
        return t

    def register_buffer(self, name: str, t: torch.Tensor) -> torch.Tensor:
        self._buffers[name] = t
        object.__setattr__(self, name, t)
        return t

    def parameters(self) -> list[torch.Tensor]:
        out = list(self._parameters.values())
        for m in self._modules.values():
            out += m.parameters()
        return out

    def train(self, mode: bool = True):
        object.__setattr__(self, "training", mode)
        for m in self._modules.values():
            m.train(mode)
        return self

    def eval(self):
        return self.train(False)

    def __call__(self, *a):
        return self.forward(*a)


class Linear(Module):
    def __init__(self, fan_in: int, fan_out: int, bias: bool = True, generator=None):
        super().__init__()
        self.register_parameter("weight", torch.randn(fan_in, fan_out, generator=generator) / fan_in ** 0.5)
        self.has_bias = bias
        if bias:
            self.register_parameter("bias", torch.zeros(fan_out))

    def forward(self, x):
        y = x @ self.weight
        return y + self.bias if self.has_bias else y


class Embedding(Module):
    def __init__(self, num: int, dim: int, generator=None):
        super().__init__()
        self.register_parameter("weight", torch.randn(num, dim, generator=generator))

    def forward(self, ix):
        return self.weight[ix]


class Flatten(Module):
    def forward(self, x):
        return x.view(x.shape[0], -1)


class FlattenConsecutive(Module):
    """(B, T, C) -> (B, T/n, C*n); squeezes the time dimension away when it becomes 1."""

    def __init__(self, n: int):
        super().__init__()
        self.n = n

    def forward(self, x):
        B, T, C = x.shape
        x = x.view(B, T // self.n, C * self.n)
        return x.squeeze(1) if x.shape[1] == 1 else x


class BatchNorm1d(Module):
    def __init__(self, dim: int, eps: float = 1e-5, momentum: float = 0.1):
        super().__init__()
        self.eps, self.momentum = eps, momentum
        self.register_parameter("gamma", torch.ones(dim))
        self.register_parameter("beta", torch.zeros(dim))
        self.register_buffer("running_mean", torch.zeros(dim))
        self.register_buffer("running_var", torch.ones(dim))

    def forward(self, x):
        if self.training:
            dims = tuple(range(x.ndim - 1))  # everything but the channel dimension
            mean, var = x.mean(dims, keepdim=True), x.var(dims, keepdim=True)
            with torch.no_grad():
                self.running_mean.mul_(1 - self.momentum).add_(self.momentum * mean.reshape(-1))
                self.running_var.mul_(1 - self.momentum).add_(self.momentum * var.reshape(-1))
        else:
            mean, var = self.running_mean, self.running_var
        return self.gamma * (x - mean) / torch.sqrt(var + self.eps) + self.beta


class Tanh(Module):
    def forward(self, x):
        return torch.tanh(x)


class Sequential(Module):
    def __init__(self, *layers: Module):
        super().__init__()
        self.layers = list(layers)
        for i, l in enumerate(layers):
            self._modules[str(i)] = l

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return x
