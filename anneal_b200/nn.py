"""Layers, activations and the SGD optimiser of anneal's ``tensor/nn`` package
(tensor/nn/nn.go), restated over ``anneal_b200.tensor``. These define the
contraction and window-reduce patterns the device has to recognise.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np

from .tensor import Tensor, broadcast_to
from .uop import dtypes
from . import uop as U


class Parameter:
    """Host-owned f32 master weights; ``load`` makes a fresh leaf for the step and
    quantises to the storage dtype (tensor/nn/nn.go:24-61)."""

    def __init__(self, shape: Sequence[int], dtype=dtypes.float32):
        self.shape, self.dtype = tuple(shape), dtype
        self.value = np.zeros(int(np.prod(shape)), dtype=np.float32)
        self.t = Tensor.new_leaf(self.shape, dtype)

    def load(self) -> Tensor:
        self.t = Tensor.new_leaf(self.shape, self.dtype).set_data(self.value)
        return self.t

    def sgd_step(self, grad: np.ndarray, lr: float) -> None:
        """value -= lr * grad in f32 on the master copy (tensor/nn/nn.go:69-76)."""
        g = np.asarray(grad, dtype=np.float32).reshape(-1)
        if g.size != self.value.size:
            raise ValueError(f"nn: SGDStep: gradient length {g.size} != parameter length {self.value.size}")
        self.value -= np.float32(lr) * g


class SGD:
    def __init__(self, params: List[Parameter], lr: float):
        self.params, self.lr = list(params), float(lr)

    def step(self, grads: Dict[Tensor, Tensor]) -> None:
        for p in self.params:
            g = grads.get(p.t)
            if g is not None:
                p.sgd_step(g.data, self.lr)


def relu(x: Tensor) -> Tensor:
    return x.maximum(Tensor.full(x.shape, 0.0, x.dtype))


def sigmoid(x: Tensor) -> Tensor:
    one = Tensor.full(x.shape, 1.0, x.dtype)
    return one.div(one.add(x.neg().exp()))


def tanh(x: Tensor) -> Tensor:
    """2*sigmoid(2x) - 1 (tensor/nn/nn.go:124-129)."""
    two = Tensor.full(x.shape, 2.0, x.dtype)
    one = Tensor.full(x.shape, 1.0, x.dtype)
    return two.mul(sigmoid(two.mul(x))).sub(one)


def gelu_tanh(x: Tensor) -> Tensor:
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), composed from the
    reference's primitives only (it has no GELU of its own). The sigmoid inside
    tanh sees max(2u, -10): in f16 storage exp(-2u) would otherwise overflow to
    inf for u < -5.5 and the backward pass would form 0 * inf."""
    k = lambda v: Tensor.full(x.shape, v, x.dtype)
    u = k(math.sqrt(2.0 / math.pi)).mul(x.add(k(0.044715).mul(x.mul(x).mul(x))))
    v = k(2.0).mul(u).maximum(k(-10.0))
    th = k(2.0).mul(sigmoid(v)).sub(k(1.0))
    return k(0.5).mul(x).mul(k(1.0).add(th))


class Linear:
    """y = x @ W^T + b, W: [out, in] (tensor/nn/nn.go:133-171)."""

    def __init__(self, in_features: int, out_features: int, bias=True, dtype=dtypes.float32):
        self.weight = Parameter((out_features, in_features), dtype)
        self.bias = Parameter((out_features,), dtype) if bias else None

    def forward(self, x: Tensor) -> Tensor:
        out = x.matmul(self.weight.t.permute((1, 0)))
        if self.bias is not None:
            out = out.add(broadcast_to(self.bias.t, out.shape))
        return out

    def params(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])


class Conv2d:
    """Stride-1 2-D convolution as an im2col built from K padded slices summed,
    then one batched matmul (tensor/nn/nn.go:173-310)."""

    def __init__(self, cin, cout, kernel, stride=(1, 1), pad=(0, 0), bias=True, dtype=dtypes.float32):
        self.weight = Parameter((cout, cin, kernel[0], kernel[1]), dtype)
        self.bias = Parameter((cout,), dtype) if bias else None
        self.stride, self.pad = tuple(stride), tuple(pad)

    def forward(self, x: Tensor) -> Tensor:
        N, Cin, H, W = x.shape
        Cout, _, kH, kW = self.weight.t.shape
        pH, pW = self.pad
        sH, sW = self.stride
        if H + 2 * pH < kH or W + 2 * pW < kW:
            raise ValueError("tensor/nn: Conv2d: kernel larger than padded input")
        Ho, Wo = H + 2 * pH - kH + 1, W + 2 * pW - kW + 1
        padded = x.pad(((0, 0), (0, 0), (pH, pH), (pW, pW))) if (pH or pW) else x
        K, HoWo = Cin * kH * kW, Ho * Wo
        im2col = None
        for ck in range(Cin):
            for kh in range(kH):
                for kw in range(kW):
                    k = ck * kH * kW + kh * kW + kw
                    patch = padded.shrink(((0, N), (ck, ck + 1), (kh, kh + Ho), (kw, kw + Wo)))
                    col = patch.reshape((N, HoWo, 1)).pad(((0, 0), (0, 0), (k, K - 1 - k)))
                    im2col = col if im2col is None else im2col.add(col)
        w_flat = self.weight.t.reshape((Cout, K)).permute((1, 0))
        out = im2col.matmul(w_flat).permute((0, 2, 1)).reshape((N, Cout, Ho, Wo))
        if self.bias is not None:
            out = out.add(self.bias.t.reshape((1, Cout, 1, 1)).expand((N, Cout, Ho, Wo)))
        if sH > 1 or sW > 1:
            out = max_pool2d(out, 1, 1, sH, sW)
        return out

    def params(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])


def max_pool2d(x: Tensor, kH: int, kW: int, sH: int, sW: int) -> Tensor:
    """Non-overlapping windows: reshape/permute then MAX over the window axis;
    overlapping: a MAXIMUM chain over kernel offsets (tensor/nn/nn.go:312-401)."""
    if x.rank != 4:
        raise ValueError(f"MaxPool2D: input must be rank 4, got rank {x.rank}")
    if kH <= 0 or kW <= 0 or sH <= 0 or sW <= 0:
        raise ValueError("MaxPool2D: kernel size and stride must be positive")
    N, C, H, W = x.shape
    if H < kH or W < kW:
        raise ValueError("MaxPool2D: input smaller than kernel")
    oH, oW = (H - kH) // sH + 1, (W - kW) // sW + 1
    if kH <= sH and kW <= sW:
        xs = x.shrink(((0, N), (0, C), (0, oH * sH), (0, oW * sW)))
        xr = xs.reshape((N, C, oH, sH, oW, sW))
        xr = xr.shrink(((0, N), (0, C), (0, oH), (0, kH), (0, oW), (0, kW)))
        xf = xr.permute((0, 1, 2, 4, 3, 5)).reshape((N, C, oH, oW, kH * kW))
        return xf.max([4])
    res = None
    for di in range(kH):
        for dj in range(kW):
            sl = x.shrink(((0, N), (0, C), (di, di + oH * sH), (dj, dj + oW * sW)))
            if sH != 1 or sW != 1:
                sl = sl.reshape((N, C, oH, sH, oW, sW)).shrink(
                    ((0, N), (0, C), (0, oH), (0, 1), (0, oW), (0, 1))).reshape((N, C, oH, oW))
            res = sl if res is None else res.maximum(sl)
    return res


def softmax_rows(x: Tensor):
    """Row softmax from primitives, with the reduced axis restored by reshape
    before each expand (a kept dimension would mis-derive EXPAND's backward,
    tensor/reduce.go:36-49 against tensor/gradient_ruleset.go:207-233)."""
    n, c = x.shape
    m = x.max([1]).reshape((n, 1)).expand((n, c))
    e = x.sub(m).exp()
    s = e.sum([1]).reshape((n, 1)).expand((n, c))
    return e.div(s)


def cross_entropy_onehot(logits: Tensor, onehot: Tensor, reduction: str = "mean") -> Tensor:
    """Softmax cross-entropy against one-hot rows, a scalar:
    -sum(onehot * (x - m - log s)) / B for "mean", without the division for "sum".
    The mean scales each term before summing, so an f16 result cannot overflow.

    The logits are materialised first. The backward of the row max compares each logit with the
    max; if the logits were an inlined f16 expression (matmul + bias) the max kernel would evaluate
    it widened to f32 inside its reduction (codegen/lower.go:158-171) while the stored max is
    rounded to f16, no element would compare equal, the tie count would be 0 and the gradient
    inf. Reading one stored copy makes both sides the same value."""
    logits = logits.contiguous()
    n, c = logits.shape
    m = logits.max([1]).reshape((n, 1)).expand((n, c))
    z = logits.sub(m)
    s = z.exp().sum([1]).reshape((n, 1)).expand((n, c))
    terms = onehot.mul(z.sub(s.log()))
    if reduction == "mean":
        terms = terms.mul(Tensor.full((n, c), 1.0 / n, terms.dtype))
    return terms.sum().neg()
