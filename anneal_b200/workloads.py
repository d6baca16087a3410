"""The five benchmark configurations as tensor graphs, with their seeded inputs.

Inputs come from a counter-based generator (splitmix64 of seed, tensor id and
element index) so that every consumer — CPU checker, CUDA path, any rank —
regenerates identical bytes without sharing files: U[0,1) from the top 24 bits,
N(0,1) by Box–Muller, Kaiming-uniform U(-b, b) with b = sqrt(6 / fan_in),
labels = u64 % classes fed as one-hot float rows (the reference has no integer
gather). The reference's own examples draw from Go's math/rand, which cannot be
reproduced outside Go; these stand in for them with the same shapes.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import nn
from . import uop as U
from .gradient import backward
from .tensor import Tensor
from .uop import dtypes

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = x
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def _stream(seed: int, tensor_id: int, n: int, lane: int = 0) -> np.ndarray:
    with np.errstate(over="ignore"):
        base = _splitmix64(np.array([seed * 0x1000003 + tensor_id * 0x10001 + lane * 0x7F4A7C15], dtype=np.uint64))[0]
        idx = np.arange(n, dtype=np.uint64)
        return _splitmix64(idx * np.uint64(0xD1342543DE82EF95) + base)


def uniform(seed: int, tensor_id: int, n: int) -> np.ndarray:
    """U[0,1) with 24 random bits, float32."""
    return ((_stream(seed, tensor_id, n) >> np.uint64(40)).astype(np.float32)) * np.float32(1.0 / (1 << 24))


def normal(seed: int, tensor_id: int, n: int) -> np.ndarray:
    u1 = ((_stream(seed, tensor_id, n, 0) >> np.uint64(40)).astype(np.float64) + 1.0) / float(1 << 24)   # (0,1]
    u2 = (_stream(seed, tensor_id, n, 1) >> np.uint64(40)).astype(np.float64) / float(1 << 24)
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * math.pi * u2)).astype(np.float32)


def kaiming_uniform(seed: int, tensor_id: int, shape) -> np.ndarray:
    fan_in = int(np.prod(shape[1:])) if len(shape) > 1 else int(shape[0])
    b = math.sqrt(6.0 / fan_in)
    n = int(np.prod(shape))
    return ((uniform(seed, tensor_id, n) * np.float32(2.0) - np.float32(1.0)) * np.float32(b)).astype(np.float32)


def labels_onehot(seed: int, tensor_id: int, n: int, classes: int) -> np.ndarray:
    lab = (_stream(seed, tensor_id, n) % np.uint64(classes)).astype(np.int64)
    oh = np.zeros((n, classes), dtype=np.float32)
    oh[np.arange(n), lab] = 1.0
    return oh.reshape(-1)


@dataclass
class TrainGraph:
    """One training step's graph: what to realize and how to feed it."""
    loss: Tensor
    params: List[nn.Parameter]
    grads: List[Tensor]
    inputs: Dict[str, Tensor]
    grad_scale: float = 1.0      # multiply gradients by this before the update (loss scaling)

    def targets(self) -> List[Tensor]:
        return [self.loss] + self.grads


def _init_params(params: List[nn.Parameter], seed: int) -> None:
    for i, p in enumerate(params):
        if len(p.shape) > 1:
            p.value[:] = kaiming_uniform(seed, 100 + i, p.shape)
        else:
            p.value[:] = 0.0


# ── C1: MLP 784→128→10, batch 64, f32 ─────────────────────────────────────────
class MLP:
    """Shape of examples/mlp.go scaled to 784→128→10 with ReLU and softmax
    cross-entropy; SGD lr 0.01."""
    seed, batch, lr = 0, 64, 0.01

    def __init__(self, batch: Optional[int] = None, dims=(784, 128, 10), dtype=dtypes.float32):
        self.batch = batch or self.batch
        self.dims, self.dtype = dims, dtype
        self.l1 = nn.Linear(dims[0], dims[1], True, dtype)
        self.l2 = nn.Linear(dims[1], dims[2], True, dtype)
        self.params = self.l1.params() + self.l2.params()
        _init_params(self.params, self.seed)
        self.x = uniform(self.seed, 1, self.batch * dims[0])
        self.y = labels_onehot(self.seed, 2, self.batch, dims[2])

    def graph(self) -> TrainGraph:
        x = Tensor.new_leaf((self.batch, self.dims[0]), self.dtype).set_data(self.x)
        y = Tensor.new_leaf((self.batch, self.dims[2]), self.dtype).set_data(self.y)
        leaves = [p.load() for p in self.params]
        logits = self.l2.forward(nn.relu(self.l1.forward(x)))
        loss = nn.cross_entropy_onehot(logits, y)
        g = backward(loss, leaves)
        return TrainGraph(loss, self.params, [g[l] for l in leaves], {"x": x, "y": y})


# ── C2: small CNN, batch 32, f32 ─────────────────────────────────────────────
class SmallCNN:
    """Conv(1→8,3x3,pad 1) ReLU MaxPool2 Conv(8→16,3x3,pad 1) ReLU MaxPool2 flatten Linear(784→10)."""
    seed, batch, lr = 1, 32, 0.01

    def __init__(self, batch: Optional[int] = None, hw: int = 28, c1: int = 8, c2: int = 16):
        self.batch = batch or self.batch
        self.hw = hw
        self.conv1 = nn.Conv2d(1, c1, (3, 3), pad=(1, 1))
        self.conv2 = nn.Conv2d(c1, c2, (3, 3), pad=(1, 1))
        self.flat = c2 * (hw // 4) * (hw // 4)
        self.fc = nn.Linear(self.flat, 10)
        self.params = self.conv1.params() + self.conv2.params() + self.fc.params()
        _init_params(self.params, self.seed)
        self.x = uniform(self.seed, 1, self.batch * hw * hw)
        self.y = labels_onehot(self.seed, 2, self.batch, 10)

    def graph(self) -> TrainGraph:
        x = Tensor.new_leaf((self.batch, 1, self.hw, self.hw)).set_data(self.x)
        y = Tensor.new_leaf((self.batch, 10)).set_data(self.y)
        leaves = [p.load() for p in self.params]
        h = nn.max_pool2d(nn.relu(self.conv1.forward(x)), 2, 2, 2, 2)
        h = nn.max_pool2d(nn.relu(self.conv2.forward(h)), 2, 2, 2, 2)
        logits = self.fc.forward(h.reshape((self.batch, self.flat)))
        loss = nn.cross_entropy_onehot(logits, y)
        g = backward(loss, leaves)
        return TrainGraph(loss, self.params, [g[l] for l in leaves], {"x": x, "y": y})


# ── C3: softmax forward+backward over [N, C], f32 ────────────────────────────
class SoftmaxFwdBwd:
    """y = softmax(x, -1); loss = sum(y * g); realizes dx (and optionally loss)."""
    seed = 2

    def __init__(self, n: int = 8192, c: int = 8192):
        self.n, self.c = n, c
        self.x = normal(self.seed, 1, n * c)
        self.g = normal(self.seed, 2, n * c)

    def graph(self, with_loss: bool = False):
        x = Tensor.new_leaf((self.n, self.c)).set_data(self.x)
        g = Tensor.new_leaf((self.n, self.c)).set_data(self.g)
        y = nn.softmax_rows(x)
        loss = y.mul(g).sum()
        dx = backward(loss, [x])[x]
        return ([dx, loss] if with_loss else [dx]), {"x": x, "g": g}

    def reference_dx(self) -> np.ndarray:
        """float64 closed form: dx = y * (g - sum(y*g))."""
        x = self.x.reshape(self.n, self.c).astype(np.float64)
        g = self.g.reshape(self.n, self.c).astype(np.float64)
        e = np.exp(x - x.max(1, keepdims=True))
        y = e / e.sum(1, keepdims=True)
        return y * (g - (y * g).sum(1, keepdims=True))


# ── C4: data-parallel wide MLP, f16 storage / f32 accumulation ───────────────
class WideMLP:
    """4 × Linear(width→width) with GELU(tanh) between, then Linear(width→classes);
    every leaf is f16, reductions accumulate in f32; SGD lr 1e-3."""
    seed, lr = 3, 1e-3

    def __init__(self, batch: int = 8192, width: int = 4096, classes: int = 1000, depth: int = 4,
                 dtype=dtypes.float16, rank: int = 0):
        self.batch, self.width, self.classes, self.depth, self.dtype, self.rank = batch, width, classes, depth, dtype, rank
        self.layers = [nn.Linear(width, width, True, dtype) for _ in range(depth)] + [nn.Linear(width, classes, True, dtype)]
        self.params = [p for l in self.layers for p in l.params()]
        _init_params(self.params, self.seed)

    def make_inputs(self):
        x = normal(self.seed, 1 + 16 * self.rank, self.batch * self.width)
        y = labels_onehot(self.seed, 2 + 16 * self.rank, self.batch, self.classes)
        return x, y

    def graph(self, x_data=None, y_data=None, loss_scale: float = 1.0) -> TrainGraph:
        x = Tensor.new_leaf((self.batch, self.width), self.dtype)
        y = Tensor.new_leaf((self.batch, self.classes), self.dtype)
        if x_data is not None:
            x.set_data(x_data)
            y.set_data(y_data)
        leaves = [p.load() for p in self.params]
        h = x
        for l in self.layers[:-1]:
            h = nn.gelu_tanh(l.forward(h))
        logits = self.layers[-1].forward(h)
        # f16 gradients of a batch mean underflow (softmax/B ~ 1e-7): differentiate the batch SUM
        # and fold 1/B into the optimiser step; report the mean
        loss = nn.cross_entropy_onehot(logits, y, "mean")
        g = backward(nn.cross_entropy_onehot(logits, y, "sum"), leaves)
        return TrainGraph(loss, self.params, [g[l] for l in leaves], {"x": x, "y": y}, 1.0 / self.batch)


# ── C5: symbolic-batch MLP under JIT (shape of examples/dynmlp.go) ───────────
class DynMLP:
    """1024→4096 ReLU →1024, MSE against y; batch bound per call."""
    seed = 4

    def __init__(self, din: int = 1024, hidden: int = 4096, dout: int = 1024, max_batch: int = 65536):
        self.din, self.hidden, self.dout = din, hidden, dout
        self.var = U.Var("n", 1, max_batch)
        self.l1 = nn.Linear(din, hidden)
        self.l2 = nn.Linear(hidden, dout)
        self.params = self.l1.params() + self.l2.params()
        _init_params(self.params, self.seed)

    def inputs(self, b: int):
        return normal(self.seed, 1, b * self.din), normal(self.seed, 2, b * self.dout)

    def graph(self, b: int, x_data=None, y_data=None):
        """Returns (forward output, loss-sum gradients) with the batch axis symbolic."""
        x = Tensor.new_symbolic_batch_input(self.var, (self.din,))
        y = Tensor.new_symbolic_batch_input(self.var, (self.dout,))
        if x_data is not None:
            x.set_data(x_data)
            y.set_data(y_data)
        leaves = [p.load() for p in self.params]
        out = self.l2.forward(nn.relu(self.l1.forward(x)))
        d = out.sub(y)
        loss = d.mul(d).sum()          # squared-error sum; the caller divides by b*dout
        g = backward(loss, leaves)
        return out, loss, [g[l] for l in leaves], {"x": x, "y": y}
