"""Full-batch gradient descent for micrograd models, returning the loss history
(nn/micrograd/train.py:4-30 of the reference)."""
from __future__ import annotations

from .value import Value


def train(model, X, y, loss_fn, epochs=100, learning_rate=0.01, verbose=False):
    losses = []
    for epoch in range(epochs):
        total_loss = Value(0)
        for xi, yi in zip(X, y):
            inputs = [x if isinstance(x, Value) else Value(x) for x in xi]
            target = yi if isinstance(yi, Value) else Value(yi)
            total_loss = total_loss + loss_fn(model(inputs), target)
        losses.append(total_loss.data)
        for p in model.parameters():
            p.grad = 0.0
        total_loss.backward()
        for p in model.parameters():
            p.data -= learning_rate * p.grad
        if verbose and (epoch % 10 == 0 or epoch == epochs - 1):
            print(f"Epoch {epoch}: loss = {total_loss.data:.6f}")
    return losses
