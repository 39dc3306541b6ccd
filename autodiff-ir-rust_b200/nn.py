"""Mirror of the reference's `nn` helpers that the configs and known-answer tests use:
Linear / LinearWithWeights (src/nn/linear.rs:5-49), Sequential (src/nn/sequential.rs),
Sigmoid / ReLU / Softmax (src/nn/activations), RMS / LayerNorm (src/nn/norm) and SGD
(src/nn/optimizers/sgd.rs:3-28), plus the two helpers upstream lists as missing (mse_loss, Tensor.abs).  Each `f` composes Tensor ops exactly as upstream does,
so the IR reaching the device has the same shape.
"""
from __future__ import annotations

import numpy as np

from . import autodiff
from .autodiff import Tensor, f32


class Module:
    def params(self) -> list:
        return []

    def f(self, x: Tensor) -> Tensor:
        raise NotImplementedError


class Linear(Module):
    """`res = dot(x, w); res += b` (src/nn/linear.rs:20-28).  `Linear(inp, out, bias)` draws
    standard-normal weights like upstream; pass `rng` for a seeded draw."""

    def __init__(self, inp=None, out=None, bias=True, *, w: Tensor = None, b: Tensor = None, rng=None):
        if w is None:
            w = autodiff.randn([inp, out], rng)
            b = autodiff.randn([out], rng) if bias else None
        self.w, self.b = w, b

    def params(self):
        return [self.w, self.b] if self.b is not None else [self.w]

    def f(self, x):
        res = autodiff.dot(x, self.w)
        if self.b is not None:
            res += self.b
        return res


def LinearWithWeights(w: Tensor, b: Tensor | None) -> Linear:
    if b is not None:
        assert b.dim()[0] == w.dim()[1], "weight dim [a,b] must match bias dim [b]"
    return Linear(w=w, b=b)


class Sigmoid(Module):
    def f(self, x):
        return f32(1.0) / (f32(1.0) + (-x).exp())


class ReLU(Module):
    def f(self, x):
        return x * x.more_than(autodiff.constant(0.0, x.dim()))


class Softmax(Module):
    def __init__(self, dim):
        self.dim = dim

    def f(self, x):
        return x.exp() / x.exp().sum(self.dim)


class RMS(Module):
    def __init__(self, d_model):
        self.scale = autodiff.ones([d_model])

    def params(self):
        return [self.scale]

    def f(self, x):
        eps = f32(1e-9)
        var = x.pow2().mean(-1).unsqueeze(-1) + eps
        return self.scale * (x / var.sqrt())


class LayerNorm(Module):
    def __init__(self, d_model):
        self.scale = autodiff.ones([d_model])
        self.bias = autodiff.zeros([d_model])

    def params(self):
        return [self.scale]

    def f(self, x):
        eps = f32(1e-9)
        y = (x - x.mean(-1).unsqueeze(-1)) / (x.var(-1, 0) + eps).sqrt().unsqueeze(-1)
        return y * self.scale + self.bias


def mse_loss(y: Tensor, target: Tensor) -> Tensor:
    """mean((y - target)^2) over every element, as a [1]-shaped tensor: the composition the reference's examples
    spell out by hand (`MSE` is on its to-do list, TODO.md:12): square, sum the axes from the last to the first,
    scale by the host-computed 1 / count."""
    d = y - target
    count = int(np.prod(d.dim()))
    s = d.pow2()
    while len(s.dim()) > 1:
        s = s.sum(len(s.dim()) - 1)
    return s.sum(0) * f32(1.0 / count)


class MSELoss(Module):
    def f(self, x: Tensor, target: Tensor = None) -> Tensor:
        return mse_loss(x, target)


class Sequential(Module):
    def __init__(self):
        self.n: list[Module] = []

    def insert(self, m: Module):
        self.n.append(m)

    def params(self):
        out = []
        for m in self.n:
            out.extend(m.params())
        return out

    def f(self, x):
        for m in self.n:
            x = m.f(x)
        return x


class SGD:
    """`p -= lr * p.grad(); p.forward()` per parameter (src/nn/optimizers/sgd.rs:9-14)."""

    def __init__(self, params, lr):
        self.n = list(params)
        self.lr = f32(lr)

    def step(self):
        for p in self.n:
            p -= self.lr * p.grad().to_node()
            p.forward()

    def zero_grad(self):
        for p in self.n:
            p.reset_grad()
