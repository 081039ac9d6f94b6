"""`Value`: a scalar that records how it was computed and can back-propagate.

Same surface as the reference's pure-Python class (nn/micrograd/value.py:5-161): `data`,
`grad`, `label`, `_children`, `_op`; operators + * ** neg - / with reflected forms; `tanh`,
`relu`, `sigmoid`, `exp`, `log`, `abs`; `backward()`. The graph, the values and the gradient
sweep live in the native engine (csrc/cpu/micrograd.cpp); this class is a handle plus the
Python-side bookkeeping (`_children` keeps operands alive, `_op` names the operation).
If the host library has not been built, an equivalent pure-Python engine is used.
"""
from __future__ import annotations

import ctypes
import math

_OPS = {"+": 1, "*": 2, "**": 3, "tanh": 4, "relu": 5, "sigmoid": 6, "exp": 7, "log": 8, "abs": 9, "/": 10}


def _load():
    try:
        from ..ops import _lib
        lib = _lib.host_lib()
    except Exception:
        return None
    lib.mg_leaf.restype = ctypes.c_int32
    lib.mg_leaf.argtypes = [ctypes.c_double]
    lib.mg_op.restype = ctypes.c_int32
    lib.mg_op.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_double]
    for name in ("mg_get_data", "mg_get_grad"):
        getattr(lib, name).restype = ctypes.c_double
        getattr(lib, name).argtypes = [ctypes.c_int32]
    for name in ("mg_set_data", "mg_set_grad"):
        getattr(lib, name).restype = None
        getattr(lib, name).argtypes = [ctypes.c_int32, ctypes.c_double]
    lib.mg_release.restype = None
    lib.mg_release.argtypes = [ctypes.c_int32]
    lib.mg_backward.restype = ctypes.c_int32
    lib.mg_backward.argtypes = [ctypes.c_int32]
    lib.mg_live_nodes.restype = ctypes.c_int32
    lib.mg_affine.restype = ctypes.c_int32
    lib.mg_affine.argtypes = [ctypes.c_int32, ctypes.POINTER(ctypes.c_int32),
                              ctypes.POINTER(ctypes.c_int32), ctypes.c_int32]
    return lib


_LIB = _load()
BACKEND = "native" if _LIB is not None else "python"


class Value:
    __slots__ = ("_id", "label", "_children", "_op", "_aux", "_pdata", "_pgrad")

    def __init__(self, data, label="", _children=(), _op=None, _id=None, _aux=0.0):
        self.label = label
        self._children = _children
        self._op = _op
        self._aux = _aux
        if _LIB is not None:
            self._id = _LIB.mg_leaf(float(data)) if _id is None else _id
        else:
            self._id = None
            self._pdata = float(data) if not isinstance(data, (int, float)) else data
            self._pgrad = 0.0

    def __del__(self):
        if _LIB is not None and self._id is not None:
            try:
                _LIB.mg_release(self._id)
            except Exception:
                pass

    # ------------------------------------------------------------------ state
    @property
    def data(self):
        return _LIB.mg_get_data(self._id) if _LIB is not None else self._pdata

    @data.setter
    def data(self, v):
        if _LIB is not None:
            _LIB.mg_set_data(self._id, float(v))
        else:
            self._pdata = v

    @property
    def grad(self):
        return _LIB.mg_get_grad(self._id) if _LIB is not None else self._pgrad

    @grad.setter
    def grad(self, v):
        if _LIB is not None:
            _LIB.mg_set_grad(self._id, float(v))
        else:
            self._pgrad = v

    def __repr__(self):
        return f"Value(data={self.data}, label='{self.label}', grad={self.grad})"

    # ------------------------------------------------------------------ graph construction
    def _make(self, op: str, other: "Value | None" = None, aux: float = 0.0, tag: str | None = None) -> "Value":
        children = (self,) if other is None else (self, other)
        tag = tag or op
        if _LIB is not None:
            nid = _LIB.mg_op(_OPS[op], self._id, -1 if other is None else other._id, float(aux))
            if nid < 0:
                raise RuntimeError("micrograd engine rejected the operation")
            return Value(0.0, "", children, tag, _id=nid, _aux=aux)
        x = self._pdata
        y = other._pdata if other is not None else None
        out = {"+": lambda: x + y, "*": lambda: x * y, "/": lambda: x / y, "**": lambda: x ** aux,
               "tanh": lambda: math.tanh(x), "relu": lambda: x if x > 0 else 0.0,
               "sigmoid": lambda: 1 / (1 + math.exp(-x)), "exp": lambda: math.exp(x),
               "log": lambda: math.log(x), "abs": lambda: abs(x)}[op]()
        return Value(out, "", children, tag, _aux=aux)

    def backward(self):
        if _LIB is not None:
            if _LIB.mg_backward(self._id) < 0:
                raise RuntimeError("backward on a released node")
            return
        # pure-Python engine: iterative post-order, then reverse sweep
        visited, seq, stack = set(), [], [self]
        while stack:
            n = stack[-1]
            if n in visited:
                stack.pop()
                continue
            pending = [c for c in n._children if c not in visited]
            if pending:
                stack.extend(pending)
            else:
                visited.add(n)
                seq.append(stack.pop())
        self._pgrad = 1.0
        for n in reversed(seq):
            g, op = n._pgrad, n._op
            if op is None:
                continue
            a = n._children[0]
            if op == "+":
                a._pgrad += g
                n._children[1]._pgrad += g
            elif op == "*":
                b = n._children[1]
                a._pgrad += g * b._pdata
                b._pgrad += g * a._pdata
            elif op == "/":
                b = n._children[1]
                a._pgrad += g / b._pdata
                b._pgrad += g * (-a._pdata / b._pdata ** 2)
            elif op.startswith("**"):
                a._pgrad += g * n._aux * a._pdata ** (n._aux - 1)
            elif op == "tanh":
                a._pgrad += g * (1 - n._pdata ** 2)
            elif op == "relu":
                a._pgrad += g * (1.0 if n._pdata > 0 else 0.0)
            elif op == "sigmoid":
                a._pgrad += g * n._pdata * (1 - n._pdata)
            elif op == "exp":
                a._pgrad += g * n._pdata
            elif op == "log":
                a._pgrad += g / a._pdata
            elif op == "abs":
                a._pgrad += g * (1.0 if a._pdata > 0 else (-1.0 if a._pdata < 0 else 0.0))
            elif op == "affine":
                kids = n._children
                fan_in = (len(kids) - 1) // 2
                for w, x in zip(kids[:fan_in], kids[fan_in:2 * fan_in]):
                    wd, xd = w._pdata, x._pdata
                    w._pgrad += g * xd
                    x._pgrad += g * wd
                kids[-1]._pgrad += g

    # ------------------------------------------------------------------ arithmetic
    @staticmethod
    def _wrap(x) -> "Value":
        return x if isinstance(x, Value) else Value(x)

    def __add__(self, other):
        return self._make("+", self._wrap(other))

    def __radd__(self, other):
        return Value(other) + self

    def __mul__(self, other):
        return self._make("*", self._wrap(other))

    def __rmul__(self, other):
        return Value(other) * self

    def __pow__(self, other):
        assert isinstance(other, (int, float)), "only supporting int/float powers"
        return self._make("**", None, float(other), tag=f"**{other}")

    def __neg__(self):
        return self * -1

    def __sub__(self, other):
        return self + (-other)

    def __rsub__(self, other):
        return Value(other) - self

    def __truediv__(self, other):
        return self._make("/", self._wrap(other))

    def __rtruediv__(self, other):
        return Value(other) / self

    # ------------------------------------------------------------------ functions
    def tanh(self):
        return self._make("tanh")

    def relu(self):
        return self._make("relu")

    def sigmoid(self):
        return self._make("sigmoid")

    def exp(self):
        return self._make("exp")

    def log(self):
        return self._make("log")

    def abs(self):
        return self._make("abs")


def affine(weights, inputs, bias) -> Value:
    """bias + sum_i weights[i] * inputs[i] as ONE graph node (op tag "affine", children
    weights..., inputs..., bias) instead of a chain of 2n scalar nodes. Numbers are wrapped into
    leaf Values. The products are added in index order starting from the bias."""
    ws = [Value._wrap(w) for w in weights]
    xs = [Value._wrap(x) for x in inputs]
    if len(ws) != len(xs):
        raise ValueError(f"{len(ws)} weights for {len(xs)} inputs")
    b = Value._wrap(bias)
    children = (*ws, *xs, b)
    if _LIB is not None:
        n = len(ws)
        arr = ctypes.c_int32 * n
        nid = _LIB.mg_affine(n, arr(*[w._id for w in ws]), arr(*[x._id for x in xs]), b._id)
        if nid < 0:
            raise RuntimeError("micrograd engine rejected the operation")
        return Value(0.0, "", children, "affine", _id=nid)
    total = b._pdata
    for w, x in zip(ws, xs):
        total = total + w._pdata * x._pdata
    return Value(total, "", children, "affine")


def live_nodes() -> int:
    """Number of graph nodes currently held by the native engine (-1 for the Python engine)."""
    return int(_LIB.mg_live_nodes()) if _LIB is not None else -1
