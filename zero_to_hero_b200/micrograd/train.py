"""Full-batch gradient descent on a micrograd model.

Contract of the reference's helper (nn/micrograd/train.py:4-30): the loss of an epoch is the
SUM of `loss_fn(model(x), y)` over the whole set, parameters move by `-learning_rate * grad`
once per epoch, and the list of epoch losses (plain floats) is returned; `verbose` prints every
tenth epoch and the last one.

The data set is wrapped into leaf `Value`s once, before the first epoch: inputs and targets are
constants of the graph, so every epoch re-uses the same leaves and only the forward nodes are
rebuilt.
"""
from __future__ import annotations

from .value import Value


def _as_leaves(row) -> list[Value]:
    return [Value._wrap(v) for v in row]


def sgd_step(params, learning_rate: float) -> None:
    for p in params:
        p.data = p.data - learning_rate * p.grad


def train(model, X, y, loss_fn, epochs=100, learning_rate=0.01, verbose=False):
    samples = [(_as_leaves(row), Value._wrap(target)) for row, target in zip(X, y)]
    params = model.parameters()
    history: list[float] = []
    for epoch in range(epochs):
        objective = Value(0.0)
        for inputs, target in samples:
            objective = objective + loss_fn(model(inputs), target)
        history.append(objective.data)
        for p in params:
            p.grad = 0.0
        for leaves, target in samples:  # the leaves persist across epochs: clear them too
            target.grad = 0.0
            for v in leaves:
                v.grad = 0.0
        objective.backward()
        sgd_step(params, learning_rate)
        if verbose and (epoch % 10 == 0 or epoch + 1 == epochs):
            print(f"Epoch {epoch}: loss = {history[-1]:.6f}")
    return history
