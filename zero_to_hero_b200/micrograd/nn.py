"""Dense tanh networks of `Value`s, built on the engine's n-ary affine node.

Behaviour of the reference's classes (nn/micrograd/nn.py:5-42): parameters start uniform in
(-1, 1) drawn from NumPy's global generator (per neuron: its weights, then its bias), every
neuron applies tanh, a layer of width 1 hands back a bare `Value` rather than a list, and
`parameters()` lists weights before the bias, neuron by neuron, layer by layer.

The construction differs: a `Layer` owns the parameter table (one row of weights per output
plus a bias column) and evaluates an output as a single `affine` node followed by `tanh`,
i.e. two graph nodes per neuron whatever the fan-in, where a chain of scalar multiply-adds
would take 2 * fan_in + 1. `Neuron` is a one-row layer kept for API parity.
"""
from __future__ import annotations

import numpy as np

from .value import Value, affine


def _draw_row(fan_in: int) -> tuple[list[Value], Value]:
    """fan_in weights and one bias, consuming the global NumPy stream in that order."""
    raw = np.random.uniform(-1, 1, size=fan_in + 1)
    return [Value(float(r)) for r in raw[:fan_in]], Value(float(raw[fan_in]))


class Layer:
    """`width` tanh units over `fan_in` inputs."""

    def __init__(self, fan_in: int, width: int):
        self.fan_in, self.width = fan_in, width
        self.weight: list[list[Value]] = []
        self.bias: list[Value] = []
        for _ in range(width):
            w, b = _draw_row(fan_in)
            self.weight.append(w)
            self.bias.append(b)

    def unit(self, k: int, x) -> Value:
        return affine(self.weight[k], x, self.bias[k]).tanh()

    def __call__(self, x):
        x = list(x) if not isinstance(x, Value) else [x]
        out = [self.unit(k, x) for k in range(self.width)]
        return out[0] if self.width == 1 else out

    def parameters(self) -> list[Value]:
        flat: list[Value] = []
        for w, b in zip(self.weight, self.bias):
            flat.extend(w)
            flat.append(b)
        return flat

    @property
    def neurons(self) -> list["Neuron"]:
        return [Neuron._view(self, k) for k in range(self.width)]

    def zero_grad(self) -> None:
        for p in self.parameters():
            p.grad = 0.0


class Neuron:
    """A single tanh unit; `w` and `b` are its weights and bias."""

    def __init__(self, fan_in: int):
        self._layer, self._k = Layer(fan_in, 1), 0

    @classmethod
    def _view(cls, layer: Layer, k: int) -> "Neuron":
        self = cls.__new__(cls)
        self._layer, self._k = layer, k
        return self

    @property
    def w(self) -> list[Value]:
        return self._layer.weight[self._k]

    @property
    def b(self) -> Value:
        return self._layer.bias[self._k]

    def __call__(self, x) -> Value:
        return self._layer.unit(self._k, list(x))

    def parameters(self) -> list[Value]:
        return [*self.w, self.b]


class MLP:
    """`MLP(n_in, [h1, h2, ..., n_out])`: a stack of `Layer`s."""

    def __init__(self, n_in: int, widths):
        dims = [n_in, *widths]
        self.layers = [Layer(a, b) for a, b in zip(dims, dims[1:])]

    def __call__(self, x):
        h = x
        for layer in self.layers:
            h = layer(h)
        return h

    def parameters(self) -> list[Value]:
        flat: list[Value] = []
        for layer in self.layers:
            flat.extend(layer.parameters())
        return flat

    def zero_grad(self) -> None:
        for layer in self.layers:
            layer.zero_grad()
