"""Lazy tensor API: the caller side of the device path.

A stand-in for anneal's ``tensor`` package (tensor/tensor.go, ops.go,
movement.go, reduce.go), kept to the same method names and graph shapes so that
the kernels reaching the device are the ones the reference scheduler would
emit: every op appends UOp nodes, nothing computes until ``realize``.

Shapes are tuples of ``int`` or ``uop.Var`` (a symbolic outermost batch
dimension, tensor/tensor.go NewSymbolicBatchInput).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import uop as U
from .uop import Op, dtypes

LN2 = math.log(2.0)
Shape = Tuple

#: host data of leaves by node id (the reference keeps it in the arena, uop/uop.go SetLeaf)
LEAF_DATA: Dict[int, np.ndarray] = {}


def _prod(xs):
    p = 1
    for x in xs:
        p *= x
    return p


def has_symbolic(sh) -> bool:
    return any(isinstance(s, U.Var) for s in sh)


class Tensor:
    __slots__ = ("node", "shape", "dtype", "data")

    def __init__(self, node: U.UOp, shape: Shape, dtype: U.DType):
        self.node, self.shape, self.dtype, self.data = node, tuple(shape), dtype, None

    # ── construction ──────────────────────────────────────────────────────
    @staticmethod
    def new_leaf(shape: Sequence[int], dtype=dtypes.float32) -> "Tensor":
        """A BUFFER leaf with a static shape (tensor/tensor.go NewLeaf)."""
        return Tensor(U.new(Op.BUFFER, dtype, (), tuple(shape)), tuple(shape), dtype)

    @staticmethod
    def new_symbolic_batch_input(var: U.Var, inner: Sequence[int], dtype=dtypes.float32) -> "Tensor":
        """A BUFFER leaf [var, *inner] whose outermost size is bound per call."""
        sh = (var,) + tuple(inner)
        return Tensor(U.new(Op.BUFFER, dtype, (), sh), sh, dtype)

    @staticmethod
    def const_scalar(v: float, dtype=dtypes.float32) -> "Tensor":
        return Tensor(U.const(dtype, v), (), dtype)

    @staticmethod
    def full(shape: Shape, v: float, dtype=dtypes.float32) -> "Tensor":
        """Scalar CONST reshaped to all-ones then expanded (tensor/tensor.go Full)."""
        t = Tensor.const_scalar(v, dtype)
        if len(shape) == 0:
            return t
        return t.reshape((1,) * len(shape)).expand(tuple(shape))

    def set_data(self, d) -> "Tensor":
        """Attach host data to a leaf; f16/bf16 leaves are quantised here, as the
        reference does at SetData (tensor/tensor.go:58-68)."""
        assert self.node.op == Op.BUFFER
        self.data = np.ascontiguousarray(U.quantize(np.asarray(d, dtype=np.float32).reshape(-1), self.dtype))
        LEAF_DATA[self.node.idx] = self.data
        return self

    @property
    def rank(self):
        return len(self.shape)

    def is_realized(self):
        return self.data is not None

    def numpy(self):
        sh = tuple(s for s in self.shape if not isinstance(s, U.Var))
        if has_symbolic(self.shape):
            return self.data.reshape((-1,) + sh)
        return self.data.reshape(self.shape)

    # ── elementwise ───────────────────────────────────────────────────────
    def cast(self, dtype) -> "Tensor":
        if dtype is self.dtype:
            return self
        return Tensor(U.new(Op.CAST, dtype, (self.node,)), self.shape, dtype)

    def _unary(self, op) -> "Tensor":
        return Tensor(U.new(op, self.dtype, (self.node,)), self.shape, self.dtype)

    def neg(self): return self._unary(Op.NEG)
    def exp2(self): return self._unary(Op.EXP2)
    def log2(self): return self._unary(Op.LOG2)
    def sin(self): return self._unary(Op.SIN)
    def sqrt(self): return self._unary(Op.SQRT)
    def recip(self): return self._unary(Op.RECIPROCAL)
    def trunc(self): return self._unary(Op.TRUNC)
    def contiguous(self): return self._unary(Op.CONTIGUOUS)

    def exp(self):
        """e^x as exp2(x * (1/ln2)) (tensor/ops.go:56-60)."""
        return self.mul(Tensor.full(self.shape, 1.0 / LN2, self.dtype)).exp2()

    def log(self):
        """ln x as log2(x) * ln2 (tensor/ops.go:62-66)."""
        return self.log2().mul(Tensor.full(self.shape, LN2, self.dtype))

    def abs(self):
        return self.maximum(self.neg())

    def _binary(self, op, other: "Tensor", out_dtype=None) -> "Tensor":
        dt = U.least_upper_dtype(self.dtype, other.dtype)
        a, b = broadcast(self.cast(dt), other.cast(dt))
        return Tensor(U.new(op, out_dtype or dt, (a.node, b.node)), a.shape, out_dtype or dt)

    def add(self, o): return self._binary(Op.ADD, o)
    def sub(self, o): return self._binary(Op.SUB, o)
    def mul(self, o): return self._binary(Op.MUL, o)
    def maximum(self, o): return self._binary(Op.MAX, o)
    def cmplt(self, o): return self._binary(Op.CMPLT, o, dtypes.bool)
    def cmpeq(self, o): return self._binary(Op.CMPEQ, o, dtypes.bool)

    def div(self, o: "Tensor") -> "Tensor":
        """Float: multiply by the reciprocal; int: IDIV (tensor/ops.go:92-98)."""
        dt = U.least_upper_dtype(self.dtype, o.dtype)
        if dt.is_float:
            return self.cast(dt).mul(o.cast(dt).recip())
        return self._binary(Op.IDIV, o)

    @staticmethod
    def where(cond: "Tensor", x: "Tensor", y: "Tensor") -> "Tensor":
        dt = U.least_upper_dtype(x.dtype, y.dtype)
        xp, yp = broadcast(x.cast(dt), y.cast(dt))
        c = broadcast_to(cond, xp.shape)
        return Tensor(U.new(Op.WHERE, dt, (c.node, xp.node, yp.node)), xp.shape, dt)

    # ── movement ──────────────────────────────────────────────────────────
    def reshape(self, new_shape) -> "Tensor":
        new_shape = tuple(new_shape)
        if new_shape == self.shape:
            return self
        if not has_symbolic(new_shape) and not has_symbolic(self.shape):
            assert _prod(new_shape) == _prod(self.shape), (self.shape, new_shape)
        return Tensor(U.new(Op.RESHAPE, self.dtype, (self.node,), new_shape), new_shape, self.dtype)

    def expand(self, new_shape) -> "Tensor":
        new_shape = tuple(new_shape)
        if new_shape == self.shape:
            return self
        assert len(new_shape) == self.rank
        for s, n in zip(self.shape, new_shape):
            assert s == n or s == 1, (self.shape, new_shape)
        return Tensor(U.new(Op.EXPAND, self.dtype, (self.node,), new_shape), new_shape, self.dtype)

    def permute(self, order) -> "Tensor":
        order = tuple(int(o) for o in order)
        assert sorted(order) == list(range(self.rank))
        sh = tuple(self.shape[o] for o in order)
        return Tensor(U.new(Op.PERMUTE, self.dtype, (self.node,), order), sh, self.dtype)

    def pad(self, padding) -> "Tensor":
        padding = tuple((int(a), int(b)) for a, b in padding)
        if all(a == 0 and b == 0 for a, b in padding):
            return self
        sh = tuple(s + a + b for s, (a, b) in zip(self.shape, padding))
        return Tensor(U.new(Op.PAD, self.dtype, (self.node,), padding), sh, self.dtype)

    def shrink(self, bounds) -> "Tensor":
        bounds = tuple((int(a), int(b)) for a, b in bounds)
        if all(a == 0 and b == s for (a, b), s in zip(bounds, self.shape)):
            return self
        sh = tuple(b - a for a, b in bounds)
        return Tensor(U.new(Op.SHRINK, self.dtype, (self.node,), bounds), sh, self.dtype)

    def flip(self, axes: Sequence[bool]) -> "Tensor":
        arg = tuple(1 if f else 0 for f in axes)
        return Tensor(U.new(Op.FLIP, self.dtype, (self.node,), arg), self.shape, self.dtype)

    def transpose(self):
        o = list(range(self.rank))
        o[-1], o[-2] = o[-2], o[-1]
        return self.permute(o)

    def flatten(self):
        return self.reshape((_prod(self.shape),))

    # ── reduce ────────────────────────────────────────────────────────────
    def _reduce(self, op, axes, keepdim) -> "Tensor":
        """REDUCE_AXIS node. The node's own shape always drops the reduced axes;
        ``keepdim`` only changes the shape the tensor handle reports
        (tensor/reduce.go:15-50)."""
        rank = self.rank
        if not axes:
            axes = list(range(rank))
        norm = sorted({a + rank if a < 0 else a for a in axes})
        assert all(0 <= a < rank for a in norm)
        out = []
        for i, s in enumerate(self.shape):
            if i not in norm:
                out.append(s)
            elif keepdim:
                out.append(1)
        node = U.new(Op.REDUCE_AXIS, self.dtype, (self.node,), (op, tuple(norm)))
        return Tensor(node, tuple(out), self.dtype)

    def sum(self, axes=None, keepdim=False): return self._reduce(Op.ADD, axes, keepdim)
    def max(self, axes=None, keepdim=False): return self._reduce(Op.MAX, axes, keepdim)

    def mean(self, axes=None, keepdim=False):
        rank = self.rank
        if not axes:
            axes = list(range(rank))
        n = _prod(self.shape[a] for a in axes)
        s = self.sum(axes, keepdim)
        dt = U.least_upper_dtype(self.dtype, dtypes.float32)
        return s.cast(dt).div(Tensor.full(s.shape, float(n), dt))

    def matmul(self, other: "Tensor") -> "Tensor":
        """A[...,M,K] @ B[...,K,N] as reshape/expand/MUL/SUM over K
        (tensor/reduce.go:105-166)."""
        a_sh, b_sh = self.shape, other.shape
        K = a_sh[-1]
        assert isinstance(K, int)
        if len(b_sh) == 1:
            assert b_sh[0] == K
            return self.mul(broadcast_to(other, a_sh)).sum([len(a_sh) - 1])
        assert b_sh[-2] == K, (a_sh, b_sh)
        a = self.reshape(a_sh + (1,))
        b = other.reshape(b_sh[:-2] + (1, K, b_sh[-1]))
        ab, bb = broadcast(a, b)
        prod = ab.mul(bb)
        return prod.sum([prod.rank - 2])


def broadcast_shapes(a: Shape, b: Shape) -> Shape:
    n = max(len(a), len(b))
    a2 = (1,) * (n - len(a)) + tuple(a)
    b2 = (1,) * (n - len(b)) + tuple(b)
    out = []
    for x, y in zip(a2, b2):
        if x == y:
            out.append(x)
        elif x == 1:
            out.append(y)
        elif y == 1:
            out.append(x)
        else:
            raise ValueError(f"tensor: incompatible shapes {a} and {b}")
    return tuple(out)


def broadcast_to(t: Tensor, target: Shape) -> Tensor:
    target = tuple(target)
    if t.rank > len(target):
        raise ValueError(f"tensor: cannot broadcast {t.shape} to {target}")
    if t.rank < len(target):
        t = t.reshape((1,) * (len(target) - t.rank) + t.shape)
    return t.expand(target)


def broadcast(a: Tensor, b: Tensor):
    sh = broadcast_shapes(a.shape, b.shape)
    return broadcast_to(a, sh), broadcast_to(b, sh)
