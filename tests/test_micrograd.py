"""micrograd: every op's value / tag / children, gradients against PyTorch, training (CPU).
Mirrors the reference's suite (nn/micrograd/tests/test_value.py, test_nn.py)."""
import math

import numpy as np
import pytest
import torch

from zero_to_hero_b200.micrograd import BACKEND, MLP, Value, live_nodes, to_dot, train


def test_native_engine_is_used_when_built():
    from zero_to_hero_b200.ops import _lib
    if (_lib._LIBDIR / "libz2h_host.so").exists():
        assert BACKEND == "native"


def test_forward_values_tags_children():
    a, b = Value(2.0, "a"), Value(3.0, "b")
    for got, data, op, kids in [(a + b, 5.0, "+", (a, b)), (a * b, 6.0, "*", (a, b)),
                                (Value(6.0) / b, 2.0, "/", None), (a ** 3, 8.0, "**3", (a,))]:
        assert got.data == data and got._op == op
        if kids:
            assert got._children == kids
    c = Value(5.0) - b
    assert c.data == 2.0 and c._op == "+" and c._children[1].data == -3.0
    n = -a
    assert n.data == -2.0 and n._op == "*" and n._children[0] is a and n._children[1].data == -1
    r = 3 + a
    assert r.data == 5.0 and r._children[0].data == 3 and r._children[1] is a
    r = 3 * a
    assert r.data == 6.0 and r._op == "*"
    r = 5 - a
    assert r.data == 3.0 and r._op == "+" and r._children[1].data == -2.0
    r = 6 / a
    assert r.data == 3.0 and r._op == "/" and r._children[1] is a
    assert a.tanh().data == pytest.approx(math.tanh(2.0)) and a.tanh()._op == "tanh"
    assert Value(-1.0).relu().data == 0.0 and a.relu().data == 2.0
    assert Value(0.0).sigmoid().data == 0.5
    assert a.exp().data == pytest.approx(math.exp(2)) and a.log().data == pytest.approx(math.log(2))
    d = Value(-3.0).abs()
    assert d.data == 3.0 and d._op == "abs"
    assert "label='a'" in repr(a)


def _composite(a, b, c):
    d = a * b
    e = d + c
    f = e - a
    g = f / 2
    h = g ** 2
    i = -h
    return i.tanh() + a.relu() * b.relu() + c.sigmoid() - a.exp() / a.log() + b.abs()


def test_backward_matches_pytorch_and_reference_constants():
    a, b, c = Value(2.0), Value(-3.0), Value(0.5)
    final = _composite(a, b, c)
    final.backward()
    ta, tb, tc = (torch.tensor(v, dtype=torch.float64, requires_grad=True) for v in (2.0, -3.0, 0.5))
    _composite(ta, tb, tc).backward()
    assert final.grad == 1.0
    for v, t in ((a, ta), (b, tb), (c, tc)):
        assert v.grad == pytest.approx(t.grad.item(), abs=1e-9)
    # the constants the reference's test hard-codes (test_value.py:214-216)
    assert a.grad == pytest.approx(-2.9704785346984863, abs=1e-6)
    assert b.grad == pytest.approx(-1.0, abs=1e-6)
    assert c.grad == pytest.approx(0.23500370979309082, abs=1e-6)


def test_gradient_accumulation_for_reused_nodes():
    a = Value(2.0)
    b = a * a
    c = b + a
    c.backward()
    assert (c.data, a.grad, b.grad, c.grad) == (6.0, 5.0, 1.0, 1.0)
    c.backward()  # gradients accumulate across calls, as in the reference
    assert a.grad == 14.0  # b.grad is 2 by now, so a gets 1 + 2 * (2 + 2) more


def test_deep_chain_does_not_recurse():
    x = Value(1.0)
    y = x
    for _ in range(20000):
        y = y + 1.0
    y.backward()
    assert x.grad == 1.0 and y.data == 20001.0


def test_nodes_are_released():
    if BACKEND != "native":
        pytest.skip("python engine")
    before = live_nodes()
    x = Value(1.0)
    y = (x * 2 + 1).tanh()
    assert live_nodes() > before
    del x, y
    import gc
    gc.collect()
    assert live_nodes() == before


def test_mlp_training_and_dot():
    np.random.seed(24)
    X = [[0, 0], [0, 1], [1, 0], [1, 1]] * 4
    y = [0, 1, 1, 0] * 4
    mlp = MLP(2, [4, 1])
    losses = train(mlp, X, y, lambda pred, target: (pred - target) ** 2, epochs=100, learning_rate=0.05)
    assert losses[-1] < losses[0]
    assert any(abs(p.grad) > 1e-6 for p in mlp.parameters())
    pred = mlp([Value(0), Value(1)])
    assert isinstance(pred, Value) and 0 < pred.data < 1
    dot = to_dot(pred)
    assert dot.startswith("\ndigraph") and "tanh" in dot and "rankdir=LR" in dot


def test_affine_node_matches_scalar_chain():
    """One n-ary node gives the value and every gradient of the multiply-add chain it replaces,
    also when a Value appears as weight and input at once."""
    from zero_to_hero_b200.micrograd.value import affine

    rng = np.random.default_rng(0)
    wv, xv, bv = rng.uniform(-1, 1, 5), rng.uniform(-1, 1, 5), 0.3
    w1, x1, b1 = [Value(v) for v in wv], [Value(v) for v in xv], Value(bv)
    w2, x2, b2 = [Value(v) for v in wv], [Value(v) for v in xv], Value(bv)
    fused = affine(w1, x1, b1).tanh()
    chain = sum((w * x for w, x in zip(w2, x2)), b2).tanh()
    assert fused._op == "tanh" and fused._children[0]._op == "affine"
    assert len(fused._children[0]._children) == 11
    assert fused.data == pytest.approx(chain.data, abs=1e-12)
    fused.backward()
    chain.backward()
    for a, b in zip(w1 + x1 + [b1], w2 + x2 + [b2]):
        assert a.grad == pytest.approx(b.grad, abs=1e-12)
    s = Value(1.5)
    sq = affine([s], [s], 0.0)  # s * s: the same node on both sides
    sq.backward()
    assert sq.data == 2.25 and s.grad == 3.0


def test_neuron_layer_api_and_parameter_order():
    from zero_to_hero_b200.micrograd import Layer, Neuron

    np.random.seed(3)
    expect = np.random.uniform(-1, 1, size=3)
    np.random.seed(3)
    n = Neuron(2)
    assert [p.data for p in n.parameters()] == pytest.approx(list(expect))
    assert len(n.w) == 2 and n.b.data == pytest.approx(expect[2])
    out = n([1.0, -2.0])
    assert out.data == pytest.approx(math.tanh(expect[0] - 2 * expect[1] + expect[2]))
    layer = Layer(3, 2)
    ys = layer([0.1, 0.2, 0.3])
    assert isinstance(ys, list) and len(ys) == 2 and len(layer.parameters()) == 8
    assert [p is q for p, q in zip(layer.neurons[1].parameters(), layer.parameters()[4:])] == [True] * 4
    assert isinstance(Layer(3, 1)([0.1, 0.2, 0.3]), Value)
